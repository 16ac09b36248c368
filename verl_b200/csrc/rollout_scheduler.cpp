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
//
// Chunked prefill: a prompt that can never fit the per-step token budget is prefilled in budget-sized chunks over several
// PREFILL steps (at most one sequence is partially prefilled at any time; the engine attends to the chunks already in the
// cache). Prefix caching: every FULL block of a prompt is named by a chain hash of the token ids it and its predecessors
// hold; blocks stay findable under that name after their last user is gone (least recently released first out when fresh
// blocks run short), and a new sequence starts from the longest run of leading blocks that is still cached. When a
// sequence finishes the engine hands over its tokens so that generated blocks become findable too (multi-turn requests
// repeat the previous turn as their prompt).
#include <algorithm>
#include <cstdint>
#include <deque>
#include <list>
#include <unordered_map>
#include <vector>

namespace {

enum SeqState : int { WAITING = 0, RUNNING = 1, FINISHED = 2, PREFILLING = 3 };
enum SeqFlags : int { NO_CHUNK = 1, NO_CACHE = 2 };
enum SchedFlags : int { CHUNKED_PREFILL = 1, PREFIX_CACHING = 2 };

inline uint64_t mix64(uint64_t h, uint64_t v) {
  h ^= v + 0x9e3779b97f4a7c15ULL + (h << 6) + (h >> 2);
  h *= 0xff51afd7ed558ccdULL;
  h ^= h >> 33;
  return h;
}

struct Seq {
  int64_t id;
  int prompt_len;       // tokens that must be prefilled before decoding (grows after a preemption)
  int num_tokens;       // tokens whose KV is (or will be after this step) in the cache
  int max_total;        // stop when num_tokens reaches this
  int state;
  int slot;             // row in the engine's static batch buffers, -1 while waiting
  int64_t share_key;    // sequences with equal non-zero key have identical prompts
  int num_preempted;
  int num_computed;     // prompt tokens whose KV is in the cache: prefix-cache hits + chunks prefilled so far
  int flags;            // SeqFlags
  int registered;       // leading blocks already offered to the prefix cache
  bool shared_user;     // counted in shared[share_key].users
  uint64_t salt;        // start value of the hash chain (distinguishes prompts whose tokens alone are ambiguous)
  std::vector<int> blocks;
  std::vector<uint64_t> hashes;   // chain hash of every full block of the tokens given to add()
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

  int sched_flags = 0;
  // prefix cache: name -> block; a cached block with no user waits in `lru` (front = first to be reused)
  std::unordered_map<uint64_t, int> cached;
  std::vector<uint64_t> hash_of;
  std::list<int> lru;
  std::vector<std::list<int>::iterator> lru_it;
  std::vector<char> in_lru;
  int64_t prefilling = -1;          // the one sequence whose prompt is partly computed
  // (sequence, tokens computed) of the step handed out last: their blocks become findable when the NEXT step is planned,
  // i.e. after the engine has issued the pass that writes them (a sequence the engine drops instead is finished first)
  std::vector<std::pair<int64_t, int>> pending;
  int64_t hit_tokens = 0, prompt_tokens = 0, chunks = 0;

  int blocks_needed(int tokens) const { return (tokens + block_size - 1) / block_size; }
  int avail() const { return (int)free_blocks.size() + (int)lru.size(); }

  int take_block() {
    int b;
    if (!free_blocks.empty()) {
      b = free_blocks.back();
      free_blocks.pop_back();
    } else if (!lru.empty()) {
      b = lru.front();
      lru.pop_front();
      in_lru[b] = 0;
      cached.erase(hash_of[b]);
      hash_of[b] = 0;
    } else {
      return -1;
    }
    refcnt[b] = 1;
    return b;
  }
  void unref(int b) {
    if (--refcnt[b] > 0) return;
    if (hash_of[b] != 0) {
      lru.push_back(b);
      lru_it[b] = std::prev(lru.end());
      in_lru[b] = 1;
    } else {
      free_blocks.push_back(b);
    }
  }
  void ref_cached(int b) {
    if (in_lru[b]) {
      lru.erase(lru_it[b]);
      in_lru[b] = 0;
    }
    refcnt[b]++;
  }
  bool alloc(Seq& s, int upto_tokens) {
    int need = blocks_needed(upto_tokens) - (int)s.blocks.size();
    if (need <= 0) return true;
    if (avail() < need) return false;
    for (int i = 0; i < need; ++i) s.blocks.push_back(take_block());
    return true;
  }
  void release(Seq& s) {
    for (int b : s.blocks) unref(b);
    s.blocks.clear();
  }
  // chain hashes of the full blocks [from_block, upto_tokens / block_size) of `tokens`, appended to s.hashes
  void extend_hashes(Seq& s, const int64_t* tokens, int upto_tokens) {
    const int nb = upto_tokens / block_size;
    for (int i = (int)s.hashes.size(); i < nb; ++i) {
      uint64_t h = i == 0 ? mix64(0x243f6a8885a308d3ULL, s.salt) : s.hashes[i - 1];
      for (int t = 0; t < block_size; ++t) h = mix64(h, (uint64_t)tokens[(size_t)i * block_size + t]);
      s.hashes.push_back(h ? h : 1);
    }
  }
  // offer the blocks that are completely computed (first `tokens_done` tokens) to the cache
  void register_blocks(Seq& s, int tokens_done) {
    if (!(sched_flags & PREFIX_CACHING) || (s.flags & NO_CACHE)) return;
    const int nb = std::min<int>({(int)s.hashes.size(), tokens_done / block_size, (int)s.blocks.size()});
    for (int i = s.registered; i < nb; ++i) {
      const int b = s.blocks[i];
      if (hash_of[b] == 0 && cached.find(s.hashes[i]) == cached.end()) {
        cached.emplace(s.hashes[i], b);
        hash_of[b] = s.hashes[i];
      }
    }
    if (nb > s.registered) s.registered = nb;
  }
  void drop_shared_user(Seq& q) {
    if (!q.shared_user) return;
    q.shared_user = false;
    auto sh = shared.find(q.share_key);
    if (sh != shared.end() && --sh->second.users <= 0) {
      for (int b : sh->second.blocks) unref(b);
      shared.erase(sh);
    }
  }
  // the prompt is completely in the cache: the sequence decodes from the next step on
  void start_decoding(Seq& q) {
    q.state = RUNNING;
    q.num_tokens = q.prompt_len;
    running.push_back(q.id);
    if (prefilling == q.id) prefilling = -1;
    if (q.share_key != 0 && q.num_preempted == 0) {
      auto sh = shared.find(q.share_key);
      if (sh == shared.end()) {
        Shared e;
        e.owner = q.id;
        e.prompt_len = q.prompt_len;
        e.users = 1;
        const int nb = blocks_needed(q.prompt_len);
        for (int i = 0; i < nb; ++i) {
          e.blocks.push_back(q.blocks[i]);
          refcnt[q.blocks[i]]++;
        }
        shared.emplace(q.share_key, std::move(e));
      } else {
        sh->second.users++;
      }
      q.shared_user = true;
    }
  }
};

}  // namespace

extern "C" {

// flags: SchedFlags (1 = chunked prefill, 2 = prefix caching)
void* vb_sched_create(int num_blocks, int block_size, int max_num_seqs, int max_batched_tokens, int flags) {
  auto* s = new Scheduler();
  s->num_blocks = num_blocks;
  s->block_size = block_size;
  s->max_num_seqs = max_num_seqs;
  s->max_batched_tokens = max_batched_tokens;
  s->sched_flags = flags;
  s->refcnt.assign(num_blocks, 0);
  s->hash_of.assign(num_blocks, 0);
  s->in_lru.assign(num_blocks, 0);
  s->lru_it.assign(num_blocks, s->lru.end());
  // block 0 is reserved as the "null" block that padded block-table entries point at
  for (int b = num_blocks - 1; b >= 1; --b) s->free_blocks.push_back(b);
  for (int i = max_num_seqs - 1; i >= 0; --i) s->free_slots.push_back(i);
  return s;
}

void vb_sched_destroy(void* h) { delete static_cast<Scheduler*>(h); }

// share_key: 0 = private prompt; equal non-zero keys mark identical prompts (GRPO samples of one prompt).
// tokens: the prompt's token ids (may be null: the sequence then takes no part in prefix caching). seq_flags: SeqFlags.
int vb_sched_add(void* h, int64_t id, int prompt_len, int max_new_tokens, int64_t share_key, const int64_t* tokens, int seq_flags,
                 uint64_t salt) {
  auto* s = static_cast<Scheduler*>(h);
  if (s->seqs.count(id)) return -1;
  if (prompt_len <= 0 || s->blocks_needed(prompt_len + max_new_tokens) > s->num_blocks - 1) return -2;
  Seq q{};
  q.id = id; q.prompt_len = prompt_len; q.num_tokens = 0; q.max_total = prompt_len + max_new_tokens;
  q.state = WAITING; q.slot = -1; q.share_key = share_key; q.num_preempted = 0;
  q.num_computed = 0; q.flags = seq_flags; q.registered = 0; q.shared_user = false; q.salt = salt;
  if (tokens == nullptr) q.flags |= NO_CACHE;
  if ((s->sched_flags & PREFIX_CACHING) && !(q.flags & NO_CACHE)) s->extend_hashes(q, tokens, prompt_len);
  s->seqs.emplace(id, std::move(q));
  s->waiting.push_back(id);
  return 0;
}

int vb_sched_num_waiting(void* h) { return (int)static_cast<Scheduler*>(h)->waiting.size(); }
int vb_sched_num_running(void* h) {
  auto* s = static_cast<Scheduler*>(h);
  return (int)s->running.size() + (s->prefilling >= 0 ? 1 : 0);
}
int vb_sched_num_free_blocks(void* h) { return static_cast<Scheduler*>(h)->avail(); }
int64_t vb_sched_num_preemptions(void* h) { return static_cast<Scheduler*>(h)->num_preemptions; }
// what: 0 = prompt tokens found in the prefix cache, 1 = prompt tokens admitted, 2 = prefill chunks beyond the first
int64_t vb_sched_counter(void* h, int what) {
  auto* s = static_cast<Scheduler*>(h);
  return what == 0 ? s->hit_tokens : what == 1 ? s->prompt_tokens : s->chunks;
}

// Plan the next step. Returns the step kind: 0 = idle, 1 = prefill, 2 = decode.
// Prefill: out_ids/out_slots describe the sequences that compute prompt tokens in this step: tokens
//          [out_starts[i], out_starts[i] + out_lens[i]) of the prompt (earlier ones are in the cache already: prefix-cache
//          hits or earlier chunks); the prompt is complete when that range ends at the prompt length.
//          out_fork_src[i] = id of the sibling whose prompt KV this sequence shares (-1: compute it), in which case
//          only block-table set-up and a copy of the partial last block are needed.
// Decode:  out_ids/out_slots = running sequences, out_lens = their kv length *including* the token decoded now.
int vb_sched_step(void* h, int64_t* out_ids, int* out_slots, int* out_lens, int64_t* out_fork_src, int* out_starts, int* out_n) {
  auto* s = static_cast<Scheduler*>(h);
  for (auto& pr : s->pending) {
    auto it = s->seqs.find(pr.first);
    if (it != s->seqs.end()) s->register_blocks(it->second, pr.second);
  }
  s->pending.clear();
  int n = 0;
  int budget = s->max_batched_tokens;
  auto emit = [&](Seq& q, int start, int len, int64_t fork_src) {
    out_ids[n] = q.id;
    out_slots[n] = q.slot;
    out_lens[n] = len;
    out_fork_src[n] = fork_src;
    out_starts[n] = start;
    ++n;
  };
  // ---- next chunk of the partly prefilled sequence
  if (s->prefilling >= 0) {
    Seq& q = s->seqs[s->prefilling];
    const int remaining = q.prompt_len - q.num_computed;
    const int chunk = std::min(remaining, budget);
    const bool last = chunk == remaining;
    if (s->alloc(q, q.num_computed + chunk + (last ? 1 : 0))) {
      emit(q, q.num_computed, chunk, -1);
      q.num_computed += chunk;
      s->pending.emplace_back(q.id, q.num_computed);
      s->chunks++;
      budget -= chunk;
      if (last) s->start_decoding(q);
    }
  }
  // ---- try to admit waiting sequences
  while (s->prefilling < 0 && budget > 0 && !s->waiting.empty() && !s->free_slots.empty()) {
    Seq& q = s->seqs[s->waiting.front()];
    int64_t fork_src = -1;
    int start = 0, chunk = q.prompt_len;
    bool last = true;
    auto sh = q.share_key != 0 && q.num_preempted == 0 ? s->shared.find(q.share_key) : s->shared.end();
    const bool can_fork = sh != s->shared.end() && sh->second.prompt_len == q.prompt_len;
    if (can_fork) {
      // share all full prompt blocks, own a private copy of the partial last block (+ room for the first new token)
      const int full = q.prompt_len / s->block_size;
      const int extra = s->blocks_needed(q.prompt_len + 1) - full;
      if (s->avail() < extra) break;
      for (int i = 0; i < full; ++i) {
        int b = sh->second.blocks[i];
        s->refcnt[b]++;
        q.blocks.push_back(b);
      }
      for (int i = 0; i < extra; ++i) q.blocks.push_back(s->take_block());
      fork_src = sh->second.owner;
      q.registered = full;
    } else {
      // longest cached run of leading blocks; at least one token is always computed (its logits start the decoding)
      int hits = 0;
      if ((s->sched_flags & PREFIX_CACHING) && !(q.flags & NO_CACHE)) {
        const int maxb = std::min<int>((int)q.hashes.size(), (q.prompt_len - 1) / s->block_size);
        while (hits < maxb && s->cached.find(q.hashes[hits]) != s->cached.end()) ++hits;
      }
      start = hits * s->block_size;
      const int remaining = q.prompt_len - start;
      chunk = remaining;
      if (remaining > budget) {
        if (n > 0) break;           // does not fit beside what is already planned: next step
        if ((s->sched_flags & CHUNKED_PREFILL) && !(q.flags & NO_CHUNK)) chunk = budget;
      }
      last = chunk == remaining;
      for (int i = 0; i < hits; ++i) {      // take the references first: the allocation below may evict unused cached blocks
        const int b = s->cached[q.hashes[i]];
        s->ref_cached(b);
        q.blocks.push_back(b);
      }
      if (!s->alloc(q, start + chunk + (last ? 1 : 0))) {
        s->release(q);
        break;
      }
      q.registered = hits;
      s->hit_tokens += start;
      s->prompt_tokens += q.prompt_len;
      budget -= chunk;
    }
    q.slot = s->free_slots.back();
    s->free_slots.pop_back();
    s->waiting.pop_front();
    emit(q, start, chunk, fork_src);
    q.num_computed = start + chunk;
    s->pending.emplace_back(q.id, q.num_computed);
    if (last) {
      s->start_decoding(q);
    } else {
      q.state = PREFILLING;
      s->prefilling = q.id;
    }
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
    s->drop_shared_user(victim);
    s->release(victim);
    s->free_slots.push_back(victim.slot);
    victim.slot = -1;
    victim.state = WAITING;
    victim.prompt_len = victim.num_tokens + 1;  // recompute prompt + every token sampled so far (the last one has no KV yet)
    victim.num_tokens = 0;
    victim.num_computed = 0;
    victim.registered = 0;
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
    out_starts[n] = 0;
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

// Remove a sequence (finished, aborted) and free its blocks and slot. tokens / n_valid (optional): the ids of the first
// n_valid tokens whose KV the cache holds for this sequence; their full blocks stay findable by later prompts.
int vb_sched_finish(void* h, int64_t id, const int64_t* tokens, int n_valid) {
  auto* s = static_cast<Scheduler*>(h);
  auto it = s->seqs.find(id);
  if (it == s->seqs.end()) return -1;
  Seq& q = it->second;
  s->pending.erase(std::remove_if(s->pending.begin(), s->pending.end(), [&](const std::pair<int64_t, int>& pr) { return pr.first == id; }),
                   s->pending.end());
  if (q.state == RUNNING && tokens != nullptr && (s->sched_flags & PREFIX_CACHING) && !(q.flags & NO_CACHE)) {
    n_valid = std::min(n_valid, q.num_tokens);
    s->extend_hashes(q, tokens, n_valid);
    s->register_blocks(q, n_valid);
  }
  if (q.state == RUNNING) {
    s->running.erase(std::find(s->running.begin(), s->running.end(), id));
    s->free_slots.push_back(q.slot);
  } else if (q.state == PREFILLING) {
    s->free_slots.push_back(q.slot);
    if (s->prefilling == id) s->prefilling = -1;
  } else {
    auto w = std::find(s->waiting.begin(), s->waiting.end(), id);
    if (w != s->waiting.end()) s->waiting.erase(w);
  }
  s->drop_shared_user(q);
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
    vb_sched_finish(h, id, nullptr, 0);
  }
  return n;
}

}  // extern "C"
