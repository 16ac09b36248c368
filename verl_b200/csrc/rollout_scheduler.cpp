// Continuous-batching scheduler and paged-KV block manager of the in-house rollout engine (host side, no CUDA).
//
// Replaces the engine core of vLLM that the reference drives through AsyncLLM
// (verl/workers/rollout/vllm_rollout/vllm_async_server.py:484-536; knobs max_num_seqs / max_num_batched_tokens /
// enable_prefix_caching in verl/trainer/config/rollout/rollout.yaml).
//
// Model: every sequence owns a list of KV blocks (block_size tokens each). A step is either a PREFILL step (admit
// waiting sequences while blocks, sequence slots and the token budget allow; sequences may be admitted as *forks* of
// a sibling with the same prompt, sharing its full prompt blocks by reference count) or a DECODE step (one token for
// every running sequence; when blocks run out the most recently admitted sequence is preempted: its blocks are
// released and it re-enters the waiting queue to be recomputed from prompt + generated tokens).
#include <algorithm>
#include <cstdint>
#include <deque>
#include <unordered_map>
#include <vector>

namespace {

enum SeqState : int { WAITING = 0, RUNNING = 1, FINISHED = 2 };

struct Seq {
  int64_t id;
  int prompt_len;       // tokens that must be prefilled before decoding (grows after a preemption)
  int num_tokens;       // tokens whose KV is (or will be after this step) in the cache
  int max_total;        // stop when num_tokens reaches this
  int state;
  int slot;             // row in the engine's static batch buffers, -1 while waiting
  int64_t share_key;    // sequences with equal non-zero key have identical prompts
  int num_preempted;
  std::vector<int> blocks;
};

struct Scheduler {
  int num_blocks, block_size, max_num_seqs, max_batched_tokens;
  std::vector<int> free_blocks;
  std::vector<int> refcnt;
  std::vector<int> free_slots;
  std::unordered_map<int64_t, Seq> seqs;
  std::deque<int64_t> waiting;
  std::vector<int64_t> running;   // admission order
  // prompts already resident: share_key -> blocks holding the prompt KV (the entry owns one reference on each)
  struct Shared { int64_t owner; std::vector<int> blocks; int prompt_len; int users; };
  std::unordered_map<int64_t, Shared> shared;
  int64_t num_preemptions = 0;

  int blocks_needed(int tokens) const { return (tokens + block_size - 1) / block_size; }

  bool alloc(Seq& s, int upto_tokens) {
    int need = blocks_needed(upto_tokens) - (int)s.blocks.size();
    if (need <= 0) return true;
    if ((int)free_blocks.size() < need) return false;
    for (int i = 0; i < need; ++i) {
      int b = free_blocks.back();
      free_blocks.pop_back();
      refcnt[b] = 1;
      s.blocks.push_back(b);
    }
    return true;
  }
  void release(Seq& s) {
    for (int b : s.blocks) {
      if (--refcnt[b] == 0) free_blocks.push_back(b);
    }
    s.blocks.clear();
  }
};

}  // namespace

extern "C" {

void* vb_sched_create(int num_blocks, int block_size, int max_num_seqs, int max_batched_tokens) {
  auto* s = new Scheduler();
  s->num_blocks = num_blocks;
  s->block_size = block_size;
  s->max_num_seqs = max_num_seqs;
  s->max_batched_tokens = max_batched_tokens;
  s->refcnt.assign(num_blocks, 0);
  // block 0 is reserved as the "null" block that padded block-table entries point at
  for (int b = num_blocks - 1; b >= 1; --b) s->free_blocks.push_back(b);
  for (int i = max_num_seqs - 1; i >= 0; --i) s->free_slots.push_back(i);
  return s;
}

void vb_sched_destroy(void* h) { delete static_cast<Scheduler*>(h); }

// share_key: 0 = private prompt; equal non-zero keys mark identical prompts (GRPO samples of one prompt).
int vb_sched_add(void* h, int64_t id, int prompt_len, int max_new_tokens, int64_t share_key) {
  auto* s = static_cast<Scheduler*>(h);
  if (s->seqs.count(id)) return -1;
  if (prompt_len <= 0 || s->blocks_needed(prompt_len + max_new_tokens) > s->num_blocks - 1) return -2;
  Seq q{};
  q.id = id; q.prompt_len = prompt_len; q.num_tokens = 0; q.max_total = prompt_len + max_new_tokens;
  q.state = WAITING; q.slot = -1; q.share_key = share_key; q.num_preempted = 0;
  s->seqs.emplace(id, std::move(q));
  s->waiting.push_back(id);
  return 0;
}

int vb_sched_num_waiting(void* h) { return (int)static_cast<Scheduler*>(h)->waiting.size(); }
int vb_sched_num_running(void* h) { return (int)static_cast<Scheduler*>(h)->running.size(); }
int vb_sched_num_free_blocks(void* h) { return (int)static_cast<Scheduler*>(h)->free_blocks.size(); }
int64_t vb_sched_num_preemptions(void* h) { return static_cast<Scheduler*>(h)->num_preemptions; }

// Plan the next step. Returns the step kind: 0 = idle, 1 = prefill, 2 = decode.
// Prefill: out_ids/out_slots/out_lens describe the admitted sequences (len = tokens to prefill);
//          out_fork_src[i] = id of the sibling whose prompt KV this sequence shares (-1: compute it), in which case
//          only block-table set-up and a copy of the partial last block are needed.
// Decode:  out_ids/out_slots = running sequences, out_lens = their kv length *including* the token decoded now.
int vb_sched_step(void* h, int64_t* out_ids, int* out_slots, int* out_lens, int64_t* out_fork_src, int* out_n) {
  auto* s = static_cast<Scheduler*>(h);
  int n = 0;
  // ---- try to admit waiting sequences
  int budget = s->max_batched_tokens;
  while (!s->waiting.empty() && !s->free_slots.empty()) {
    Seq& q = s->seqs[s->waiting.front()];
    int64_t fork_src = -1;
    auto sh = q.share_key != 0 && q.num_preempted == 0 ? s->shared.find(q.share_key) : s->shared.end();
    const bool can_fork = sh != s->shared.end() && sh->second.prompt_len == q.prompt_len;
    if (can_fork) {
      // share all full prompt blocks, own a private copy of the partial last block (+ room for the first new token)
      const int full = q.prompt_len / s->block_size;
      const int extra = s->blocks_needed(q.prompt_len + 1) - full;
      if ((int)s->free_blocks.size() < extra) break;
      for (int i = 0; i < full; ++i) {
        int b = sh->second.blocks[i];
        s->refcnt[b]++;
        q.blocks.push_back(b);
      }
      for (int i = 0; i < extra; ++i) {
        int b = s->free_blocks.back();
        s->free_blocks.pop_back();
        s->refcnt[b] = 1;
        q.blocks.push_back(b);
      }
      fork_src = sh->second.owner;
      sh->second.users++;
    } else {
      if (q.prompt_len > budget && n > 0) break;
      if (!s->alloc(q, q.prompt_len + 1)) break;
      budget -= q.prompt_len;
      if (q.share_key != 0 && q.num_preempted == 0 && s->shared.find(q.share_key) == s->shared.end()) {
        Scheduler::Shared e;
        e.owner = q.id;
        e.prompt_len = q.prompt_len;
        e.users = 1;
        const int nb = s->blocks_needed(q.prompt_len);
        for (int i = 0; i < nb; ++i) {
          e.blocks.push_back(q.blocks[i]);
          s->refcnt[q.blocks[i]]++;
        }
        s->shared.emplace(q.share_key, std::move(e));
      } else if (q.share_key != 0 && q.num_preempted == 0) {
        s->shared[q.share_key].users++;
      }
    }
    q.state = RUNNING;
    q.slot = s->free_slots.back();
    s->free_slots.pop_back();
    q.num_tokens = q.prompt_len;
    s->running.push_back(q.id);
    s->waiting.pop_front();
    out_ids[n] = q.id;
    out_slots[n] = q.slot;
    out_lens[n] = q.prompt_len;
    out_fork_src[n] = fork_src;
    ++n;
    if (budget <= 0) break;
  }
  if (n > 0) {
    *out_n = n;
    return 1;
  }
  // ---- decode step for all running sequences; preempt newest ones while blocks are missing
  if (s->running.empty()) {
    *out_n = 0;
    return 0;
  }
  size_t i = 0;
  while (i < s->running.size()) {
    Seq& q = s->seqs[s->running[i]];
    if (s->alloc(q, q.num_tokens + 1)) {
      ++i;
      continue;
    }
    // out of blocks: preempt the most recently admitted sequence (possibly q itself)
    Seq& victim = s->seqs[s->running.back()];
    if (victim.share_key != 0 && victim.num_preempted == 0) {
      auto sh = s->shared.find(victim.share_key);
      if (sh != s->shared.end() && --sh->second.users <= 0) {
        for (int b : sh->second.blocks)
          if (--s->refcnt[b] == 0) s->free_blocks.push_back(b);
        s->shared.erase(sh);
      }
    }
    s->release(victim);
    s->free_slots.push_back(victim.slot);
    victim.slot = -1;
    victim.state = WAITING;
    victim.prompt_len = victim.num_tokens + 1;  // recompute prompt + every token sampled so far (the last one has no KV yet)
    victim.num_tokens = 0;
    victim.num_preempted++;
    s->num_preemptions++;
    s->waiting.push_front(victim.id);
    s->running.pop_back();
  }
  for (int64_t id : s->running) {
    Seq& q = s->seqs[id];
    q.num_tokens += 1;
    out_ids[n] = id;
    out_slots[n] = q.slot;
    out_lens[n] = q.num_tokens;
    out_fork_src[n] = -1;
    ++n;
  }
  *out_n = n;
  return n > 0 ? 2 : 0;
}

// Copy a sequence's block list into out (up to cap entries); returns the number of blocks.
int vb_sched_blocks(void* h, int64_t id, int* out, int cap) {
  auto* s = static_cast<Scheduler*>(h);
  auto it = s->seqs.find(id);
  if (it == s->seqs.end()) return -1;
  int n = std::min<int>(cap, (int)it->second.blocks.size());
  for (int i = 0; i < n; ++i) out[i] = it->second.blocks[i];
  return (int)it->second.blocks.size();
}

int vb_sched_num_tokens(void* h, int64_t id) {
  auto* s = static_cast<Scheduler*>(h);
  auto it = s->seqs.find(id);
  return it == s->seqs.end() ? -1 : it->second.num_tokens;
}

int vb_sched_num_preempted(void* h, int64_t id) {
  auto* s = static_cast<Scheduler*>(h);
  auto it = s->seqs.find(id);
  return it == s->seqs.end() ? -1 : it->second.num_preempted;
}

// True when the sequence has produced its last allowed token (length limit); EOS is reported by the engine.
int vb_sched_at_limit(void* h, int64_t id) {
  auto* s = static_cast<Scheduler*>(h);
  auto it = s->seqs.find(id);
  if (it == s->seqs.end()) return -1;
  return it->second.num_tokens + 1 >= it->second.max_total ? 1 : 0;
}

// Remove a sequence (finished, aborted) and free its blocks and slot.
int vb_sched_finish(void* h, int64_t id) {
  auto* s = static_cast<Scheduler*>(h);
  auto it = s->seqs.find(id);
  if (it == s->seqs.end()) return -1;
  Seq& q = it->second;
  if (q.state == RUNNING) {
    s->running.erase(std::find(s->running.begin(), s->running.end(), id));
    s->free_slots.push_back(q.slot);
  } else {
    auto w = std::find(s->waiting.begin(), s->waiting.end(), id);
    if (w != s->waiting.end()) s->waiting.erase(w);
  }
  if (q.share_key != 0 && q.num_preempted == 0 && q.state != WAITING) {
    auto sh = s->shared.find(q.share_key);
    if (sh != s->shared.end() && --sh->second.users <= 0) {
      for (int b : sh->second.blocks)
        if (--s->refcnt[b] == 0) s->free_blocks.push_back(b);
      s->shared.erase(sh);
    }
  }
  s->release(q);
  s->seqs.erase(it);
  return 0;
}

// Abort everything (weight sync interrupts generation): ids of all live sequences are returned, state is cleared.
int vb_sched_abort_all(void* h, int64_t* out_ids, int cap) {
  auto* s = static_cast<Scheduler*>(h);
  std::vector<int64_t> ids;
  for (auto& kv : s->seqs) ids.push_back(kv.first);
  int n = 0;
  for (int64_t id : ids) {
    if (n < cap) out_ids[n] = id;
    ++n;
    vb_sched_finish(h, id);
  }
  return n;
}

}  // extern "C"
