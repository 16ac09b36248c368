// Persistent bf16 GEMM for sm_100a: TMA-fed shared-memory ring, tcgen05.mma with fp32 accumulators in TMEM
// (double buffered so the epilogue of tile i overlaps the main loop of tile i+1), tcgen05.ld epilogue.
//
//   C[M,N] (+)= op(A) * op(B) (+ bias)
//
// Both operands may be K-major ("row = M or N index, K contiguous": x[T,in], W[out,in]) or MN-major
// ("row = K index, M or N contiguous": dy[T,out] as A of a weight gradient, W[out,in] as B of an input
// gradient), so forward, input-gradient and weight-gradient GEMMs of a linear layer run without a transpose
// copy. Replaces the cuBLAS calls a torch nn.Linear makes under autocast in the reference
// (verl/workers/engine/fsdp/transformer_impl.py:1581-1590).
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner, warps 2-5 = epilogue
// (warp w reads TMEM lanes 32*(w%4)..+31).
#include <cstdlib>

#include "common.cuh"
#include "tma_host.h"

namespace vb {

constexpr int BM = 128;
constexpr int BK = 64;       // 64 bf16 = 128 B = one swizzle row
constexpr int UMMA_K = 16;
constexpr int A_TILE_BYTES = BM * BK * 2;

// KA: 64-element K atoms per pipeline stage. KA = 2 fetches 256 contiguous bytes of every operand row per stage (two TMA
// boxes): memory-bound decode-sized problems then touch each DRAM page in longer bursts and pay half the barrier traffic.
template <int BN, int KA = 1>
struct GemmCfg {
  static constexpr int B_TILE_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = KA * (A_TILE_BYTES + B_TILE_BYTES);
  static constexpr int MAX_STAGES = (220 * 1024) / STAGE_BYTES;
  static constexpr int STAGES = MAX_STAGES > 8 ? 8 : MAX_STAGES;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
  static constexpr int TMEM_COLS = (2 * BN) < 32 ? 32 : (2 * BN);
};

enum : int { GEMM_OUT_F32 = 1, GEMM_ACCUM = 2 };
enum : int { EPI_STORE = 0, EPI_LOGPROB = 1, EPI_DLOGITS = 2, EPI_PEER = 3 };

// Multi-GPU arguments. Operand segmentation: rows of A (seg_mode 1) or of B (seg_mode 2) are split into n_seg equal
// segments, each living in a different rank's memory and described by its own tensor map; the producer warp reads a
// tile from whichever rank owns it (plain TMA load from peer memory, no multicast) -> all-gather fused into the GEMM.
// EPI_PEER epilogue: the bf16 output tile is stored into symmetric buffers of other ranks, slot `rank` of each
// destination (all ranks when rows_per_owner == 0 -> all-reduce input; the owner of the row block otherwise ->
// reduce-scatter input). A barrier and a slot-sum kernel finish the collective.
constexpr int MAX_TP = 8;
struct DistArgs {
  int seg_mode, seg_rows, n_seg;     // seg_mode 3: A is split along K (seg_rows = K columns per rank), rows offset by row_off
  int rank, world;
  int rows_per_owner;
  long slot_elems;
  int row_off;                       // seg_mode 3: first row of this rank's block inside every peer's buffer
  int head_dim;                      // > 0: EPI_PEER routes whole heads (head_dim columns) through head_map (sequence → head a2a)
  uint16_t head_map[192];            // per output head: (destination rank << 12) | destination head slot
  void* peer_out[MAX_TP];
  // Staging of the remote part of a gathered operand: tiles that live on another rank are copied ONCE over NVLink into
  // `stage` (laid out like the gathered operand) at kernel start, in 16-row pieces dealt out over all CTAs; every piece adds one
  // to the flag of its 128-row chunk (zeroed by the launcher before the call) and the TMA producer waits until the flag of the
  // tile it is about to load has counted STAGE_PARTS pieces. Without staging every output tile would fetch its operand tile from the peer again.
  // Grouped (mixture-of-experts) GEMM. Token rows are sorted by expert and every expert's segment is padded to a multiple
  // of 128 rows, so a 128-row block belongs to exactly one expert.
  //   group_mode 1: C[rows, N] = A[rows, K] * B[e]^T with e = blk_expert[row block] (< 0: block unused, tile skipped);
  //                 tmB is a 3-D map whose outermost coordinate is the expert.
  //   group_mode 2: C[e][M, N] (+)= A[rows_e, M]^T * B[rows_e, N] over the rows of expert e (weight gradient);
  //                 expert_rng[e] = (first block, end block); the tile index runs over (expert, m block, n block).
  // Signalled all-reduce (EPI_PEER, rows_per_owner == 0): partials stay in this rank's buffer; instead of a separate barrier
  // launch, the LAST CTA of the GEMM advances this rank's epoch (sig_local[0]) and stores it into every peer's flag word for
  // this rank; the slot-sum kernel waits for the peers' flags and pulls. Buffers alternate by epoch parity, so a rank can
  // start its next GEMM while a peer still reads the previous result.
  long sig_half;                     // elements between the two slot buffers (fixed per context; slot_elems may change per call)
  int* sig_local;                    // [0] epoch, [1] finished-CTA counter, [SIG_FLAGS + p] flag written by rank p
  int* sig_peer[MAX_TP];
  int group_mode;
  int num_experts;
  const int* blk_expert;
  const int2* expert_rng;
  // Expert-parallel dispatch fused into the grouped GEMM's A operand (seg_mode 4, with group_mode 1): row r of the expert-sorted,
  // block-padded operand is row (row_src[r] & 0xFFFFFF) of rank (row_src[r] >> 24)'s token buffer seg_ptr[rank]; row_src[r] < 0 is
  // a padding row (zeros). The copy warps gather the rows of a 128-row block into `stage` while earlier blocks are multiplied.
  const int* row_src;
  // Combine fused into the epilogue (EPI_PEER with row_dst): output row r, multiplied by row_w[r], becomes row
  // (row_dst[r] & 0xFFFFFF) of rank (row_dst[r] >> 24)'s buffer peer_out[rank] (row stride ldc); row_dst[r] < 0: not stored.
  const int* row_dst;
  const float* row_w;
  int peer_lines;                    // EPI_PEER: rows leave as 128-byte bulk stores from shared-memory lines (N and head_dim multiples of 64)
  void* stage;
  int* stage_flags;
  int stage_epoch;
  int ld_stage;                      // row stride of `stage` in elements
  int ld_seg;                        // row stride of the peers' segments in elements
  const void* seg_ptr[MAX_TP];
  CUtensorMap stage_map;
  CUtensorMap seg[MAX_TP];
};

constexpr int STAGE_PARTS = 8;
constexpr int SIG_FLAGS = 16;
// shared-memory ring of the fused token dispatch: rows (or 4 KB pieces of longer rows) in flight per SM, one zeroed piece for padding rows
constexpr int DISPATCH_SLOTS = 7;
constexpr int DISPATCH_SLOT_BYTES = 4096;
constexpr int DISPATCH_SMEM_BYTES = (DISPATCH_SLOTS + 1) * DISPATCH_SLOT_BYTES + 64;
// combine epilogue: one 128-byte line (+16 bytes so that neighbouring lines start in different banks) per epilogue thread
constexpr int COMBINE_LINE_PITCH = 144;
constexpr int COMBINE_SMEM_BYTES = 128 * COMBINE_LINE_PITCH;

__device__ __forceinline__ bool stage_wait(const int* flag, int epoch, volatile int* abort_flag, int* err_word) {
  epoch = STAGE_PARTS;            // the launcher zeroes the flags before every call; every piece of a chunk adds one
  uint64_t t0 = 0;
  uint32_t n = 0;
  while (true) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v >= epoch) {
      asm volatile("fence.proxy.async;" ::: "memory");   // the staged bytes were written by ordinary stores, TMA reads them next
      return true;
    }
    if ((++n & 0x3F) == 0) {
      if (*abort_flag) return false;
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > VB_WAIT_LIMIT_NS) {
        *abort_flag = 1;
        atomicCAS(err_word, 0, VB_ERR_WAIT_PEER | (blockIdx.x << 8));
        return false;
      }
      __nanosleep(100);
    }
  }
}

// Extra epilogue inputs of the fused lm_head variants (rows = tokens, columns = vocabulary entries).
struct LmHeadEpi {
  float inv_temp;
  const long* labels;     // [M]
  int col_offset;         // global vocabulary index of column 0 of this launch (vocab-chunked backward)
  // EPI_LOGPROB: per (column tile, row) partial softmax statistics of x = logit * inv_temp
  float* part_max;        // [num_n_tiles, M]
  float* part_sum;        // sum exp(x - max)
  float* part_sumx;       // sum x * exp(x - max)
  float* label_logit;     // [M] x at the label column (written by the one tile that contains it)
  // EPI_DLOGITS: dL/dlogit = inv_temp * ( g_lp * (1[label] - p) - g_ent * p * (x - lse + H) ),  p = exp(x - lse)
  const float* lse;       // [M]
  const float* ent;       // [M]
  const float* g_lp;      // [M]
  const float* g_ent;     // [M] or null
};

// COPY_WARPS > 0 adds that many warps (after the six role warps) whose only job is to stage remote operand chunks.
template <int BN, bool A_MN, bool B_MN, int EPI, int COPY_WARPS = 0, int KA = 1>
__global__ void __launch_bounds__(192 + 32 * COPY_WARPS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, void* __restrict__ Cv,
                 const bf16* __restrict__ bias, int M, int N, int K, int ldc, int flags, int* err_word, const LmHeadEpi epi,
                 int split_k, int kb_per_split, float* __restrict__ split_ws, const __grid_constant__ DistArgs dist) {
  static_assert(KA == 1 || (!A_MN && !B_MN && COPY_WARPS == 0), "multi-atom stages: K-major operands, no staging warps");
  using Cfg = GemmCfg<BN, KA>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (M + BM - 1) / BM;
  const int num_n = (N + BN - 1) / BN;
  const int num_kb_total = (K + BK * KA - 1) / (BK * KA);      // K blocks of one pipeline stage
  // split-K: a work unit is (output tile, K slice); partial sums go to an fp32 workspace and are reduced afterwards
  const int num_tiles = dist.group_mode == 2 ? num_m * num_n * dist.num_experts : num_m * num_n * split_k;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 128);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc<Cfg::TMEM_COLS>(tmem_slot);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // signalled all-reduce: the slot buffer of this call is chosen by the parity of the epoch BEFORE this launch
  // (split-K: every K slice of every rank has a slot of its own, summed by the slot-sum kernel)
  const long sig_slot_off = (dist.sig_local != nullptr) ? (long)(dist.sig_local[0] & 1) * dist.sig_half : 0;

  // Tile order: groups of GROUP_M row-blocks sweep N together so a B column block stays in L2.
  constexpr int GROUP_M = 8;
  auto tile_coords = [&](int u, int& mb, int& nb) {
    int t = u / split_k;
    int per_group = GROUP_M * num_n;
    int g = t / per_group;
    int first_m = g * GROUP_M;
    int gsz = min(num_m - first_m, GROUP_M);
    int r = t - g * per_group;
    mb = first_m + (r % gsz);
    nb = r / gsz;
    if (dist.stage != nullptr) {       // start with the tiles whose gathered operand rows are this rank's own
      if (dist.seg_mode == 1) mb = (mb + (dist.rank * dist.seg_rows) / BM) % num_m;
      else if (dist.seg_mode == 2) nb = (nb + (dist.rank * dist.seg_rows) / BN) % num_n;
    }
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int mb, nb, expert = 0;
        int kb0, kb1;
        if (dist.group_mode == 2) {
          expert = t / (num_m * num_n);
          tile_coords(t - expert * num_m * num_n, mb, nb);
          const int2 rng = dist.expert_rng[expert];
          kb0 = rng.x * (128 / BK);
          kb1 = rng.y * (128 / BK);
          if (kb1 <= kb0) continue;
        } else {
          tile_coords(t, mb, nb);
          kb0 = (t % split_k) * kb_per_split;
          kb1 = min(num_kb_total, kb0 + kb_per_split);
          if (dist.group_mode == 1) {
            expert = dist.blk_expert[mb];
            if (expert < 0) continue;
          }
        }
        const int m0 = mb * BM, n0 = nb * BN;
        // Decode-sized problems (a few row blocks): every CTA of a row block would ask for the same A tile at the same
        // moment and queue up on one L2 slice. Start each column block at a different K step and wrap around (the order of
        // the K steps does not matter for the sum); CTAs that share a B tile keep the same order.
        const int nk = kb1 - kb0;
        const int rot = (num_m <= 4 && dist.seg_mode == 0 && dist.group_mode == 0 && nk > 1) ? (nb * 5) % nk : 0;
        for (int ki = 0; ki < nk; ++ki) {
          const int kb = kb0 + (ki + rot >= nk ? ki + rot - nk : ki + rot);
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, err_word, VB_ERR_WAIT_EMPTY)) { ok = false; break; }
          uint8_t* sa = smem + s * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + KA * A_TILE_BYTES;
          mbar_expect_tx(&full_bar[s], Cfg::STAGE_BYTES);
          const int k0 = kb * BK * KA;
          if constexpr (KA > 1) {
            // plain K-major problem: KA adjacent 64-column atoms of A and of B (columns past K read as zeros)
#pragma unroll
            for (int a = 0; a < KA; ++a) {
              tma_load_2d(sa + a * A_TILE_BYTES, &tmA, k0 + a * BK, m0, &full_bar[s]);
              tma_load_2d(sb + a * Cfg::B_TILE_BYTES, &tmB, k0 + a * BK, n0, &full_bar[s]);
            }
            if (++s == STAGES) { s = 0; ph ^= 1; }
            continue;
          }
          if (!A_MN) {
            if (dist.seg_mode == 1) {
              const int owner = m0 / dist.seg_rows;
              if (dist.stage != nullptr && owner != dist.rank) {
                if (kb == kb0 && !stage_wait(dist.stage_flags + m0 / 128, dist.stage_epoch, abort_flag, err_word)) { ok = false; break; }
                tma_load_2d(sa, &dist.stage_map, k0, m0, &full_bar[s]);
              } else {
                tma_load_2d(sa, &dist.seg[owner], k0, m0 % dist.seg_rows, &full_bar[s]);
              }
            } else if (dist.seg_mode == 4) {
              if (kb == kb0 && !stage_wait(dist.stage_flags + m0 / 128, dist.stage_epoch, abort_flag, err_word)) { ok = false; break; }
              tma_load_2d(sa, &dist.stage_map, k0, m0, &full_bar[s]);
            } else if (dist.seg_mode == 3) {
              const int owner = k0 / dist.seg_rows;
              if (dist.stage != nullptr && owner != dist.rank) {
                if (k0 % dist.seg_rows == 0 &&
                    !stage_wait(dist.stage_flags + (m0 / 128) * dist.n_seg + owner, dist.stage_epoch, abort_flag, err_word)) { ok = false; break; }
                tma_load_2d(sa, &dist.stage_map, k0, m0, &full_bar[s]);
              } else {
                tma_load_2d(sa, &dist.seg[owner], k0 % dist.seg_rows, m0 + dist.row_off, &full_bar[s]);
              }
            } else {
              tma_load_2d(sa, &tmA, k0, m0, &full_bar[s]);
            }
          } else {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i) tma_load_2d(sa + i * (BK * 128), &tmA, m0 + 64 * i, k0, &full_bar[s]);
          }
          if (!B_MN) {
            if (dist.seg_mode == 2) {
              const int owner = n0 / dist.seg_rows;
              if (dist.stage != nullptr && owner != dist.rank) {
                if (kb == kb0) {
                  bool got = true;
                  for (int c = 0; c < BN / 128 && got; ++c) got = stage_wait(dist.stage_flags + n0 / 128 + c, dist.stage_epoch, abort_flag, err_word);
                  if (BN < 128 && got) got = stage_wait(dist.stage_flags + n0 / 128, dist.stage_epoch, abort_flag, err_word);
                  if (!got) { ok = false; break; }
                }
                tma_load_2d(sb, &dist.stage_map, k0, n0, &full_bar[s]);
              } else {
                tma_load_2d(sb, &dist.seg[owner], k0, n0 % dist.seg_rows, &full_bar[s]);
              }
            } else if (dist.group_mode == 1) {
              tma_load_3d(sb, &tmB, k0, n0, expert, &full_bar[s]);
            } else {
              tma_load_2d(sb, &tmB, k0, n0, &full_bar[s]);
            }
          } else if (dist.group_mode == 1) {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i) tma_load_3d(sb + i * (BK * 128), &tmB, n0 + 64 * i, k0, expert, &full_bar[s]);
          } else {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i) tma_load_2d(sb + i * (BK * 128), &tmB, n0 + 64 * i, k0, &full_bar[s]);
          }
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BM, BN, 1, 1, A_MN, B_MN);
      int s = 0;
      uint32_t ph = 0;
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
        int kb0, kb1;
        if (dist.group_mode == 2) {
          const int2 rng = dist.expert_rng[t / (num_m * num_n)];
          kb0 = rng.x * (128 / BK);
          kb1 = rng.y * (128 / BK);
          if (kb1 <= kb0) { --it; continue; }          // skipped tiles do not consume an accumulator buffer
        } else {
          kb0 = (t % split_k) * kb_per_split;
          kb1 = min(num_kb_total, kb0 + kb_per_split);
          if (dist.group_mode == 1) {
            int mb, nb;
            tile_coords(t, mb, nb);
            if (dist.blk_expert[mb] < 0) { --it; continue; }
          }
        }
        const uint32_t acc = it & 1;
        const uint32_t acc_ph = (it >> 1) & 1;
        if (!mbar_wait(&tempty_bar[acc], acc_ph ^ 1, abort_flag, err_word, VB_ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[s], ph, abort_flag, err_word, VB_ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * Cfg::STAGE_BYTES);
          const uint32_t sb = sa + KA * A_TILE_BYTES;
#pragma unroll
          for (int k = 0; k < KA * BK / UMMA_K; ++k) {
            // K-major: 8-row groups are 1024 B apart, a K step of 16 elements is 32 B inside the swizzle row; with KA > 1 the
            //          next 64-column atom is a whole tile further.
            // MN-major: 64-element column atoms are BK*128 B apart (LBO), 8-row K groups 1024 B apart (SBO);
            //           a K step of 16 rows is 2048 B.
            const uint32_t ka_off = (KA > 1) ? (k >> 2) * A_TILE_BYTES + (k & 3) * 32 : k * 32;
            const uint32_t kb_off = (KA > 1) ? (k >> 2) * Cfg::B_TILE_BYTES + (k & 3) * 32 : k * 32;
            uint64_t ad = A_MN ? make_sdesc_sw128(sa + k * 2048, BK * 128, 1024) : make_sdesc_sw128(sa + ka_off, 16, 1024);
            uint64_t bd = B_MN ? make_sdesc_sw128(sb + k * 2048, BK * 128, 1024) : make_sdesc_sw128(sb + kb_off, 16, 1024);
            umma_f16(d_tmem, ad, bd, idesc, ((kb - kb0) | k) != 0);
          }
          umma_commit(&empty_bar[s]);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (ok) umma_commit(&tfull_bar[acc]);
      }
    }
  } else if (COPY_WARPS > 0 && warp >= 6) {
    // ------------------------------------------------------------ staging copies (dedicated warps)
    if constexpr (COPY_WARPS > 0) {
    if (dist.stage != nullptr) {
      // Bring the chunks of the gathered operand that live elsewhere into the local staging buffer, once per call, while the
      // tensor cores work on chunks that have arrived. Ordinary loads from a peer are limited by the few requests an SM may have
      // outstanding (~350 GB/s over the whole GPU, measured), so the rows travel as bulk copies: peer memory -> a ring of row
      // buffers in shared memory -> staging, issued by ONE thread per CTA with DISPATCH_SLOTS pieces of up to 4 KB in flight.
      // 128-row chunks are dealt to the CTAs round-robin in the order the tiles consume them; a chunk's flag receives all its
      // STAGE_PARTS at once when its rows have landed. Nothing here waits on another CTA, so the copies always make progress.
      //   seg_mode 1 / 2: chunk c = rows [128 c, 128 c + 128) of the row-gathered operand (own chunks are read in place);
      //   seg_mode 3:     chunk (row block, owner) = that owner's K columns of 128 rows;
      //   seg_mode 4:     token dispatch, row r of a used block comes from (rank, row) = row_src[r] (own rows too: the operand
      //                   must be contiguous for the tensor map), padding rows are zero-filled.
      constexpr int CT = 32 * COPY_WARPS;                 // copy threads per CTA
      const int et = threadIdx.x - 192;
      const bf16* const* srcs = reinterpret_cast<const bf16* const*>(dist.seg_ptr);
      bf16* stage = reinterpret_cast<bf16*>(dist.stage);
      uint8_t* bounce = smem + STAGES * Cfg::STAGE_BYTES + 256;
      uint8_t* zero_row = bounce + DISPATCH_SLOTS * DISPATCH_SLOT_BYTES;
      uint64_t* bbar = reinterpret_cast<uint64_t*>(zero_row + DISPATCH_SLOT_BYTES);
      for (int i = et; i < DISPATCH_SLOT_BYTES / 16; i += CT) reinterpret_cast<uint4*>(zero_row)[i] = make_uint4(0, 0, 0, 0);
      if (et == 0) {
        for (int j = 0; j < DISPATCH_SLOTS; ++j) mbar_init(&bbar[j], 1);
        mbar_fence_init();
      }
      asm volatile("fence.proxy.async;" ::: "memory");            // the zero row was written by ordinary stores, bulk copies read it
      asm volatile("bar.sync 1, %0;" ::"n"(CT) : "memory");
      if (et == 0) {
        const int mode = dist.seg_mode;
        const bool by_k = mode == 3;
        const int row_bytes = (by_k ? dist.seg_rows : K) * 2;
        const int nseg = (row_bytes + DISPATCH_SLOT_BYTES - 1) / DISPATCH_SLOT_BYTES;
        const int n_chunks = mode == 4 ? M / 128 : by_k ? ((M + 127) / 128) * dist.n_seg : dist.seg_rows * dist.n_seg / 128;
        uint32_t phase = 0;
        int mine = 0;
        bool ok = true;
        for (int c = 0; c < n_chunks && ok; ++c) {
          int owner = -1, row0, rows = 128;
          long dst_col = 0;
          if (mode == 4) {
            if (dist.blk_expert[c] < 0) continue;                 // unused block: the producer skips it as well
            row0 = c * 128;
          } else if (by_k) {
            const int mc = c / dist.n_seg;
            owner = c - mc * dist.n_seg;
            row0 = mc * 128;
            rows = min(128, M - row0);
            dst_col = (long)owner * dist.seg_rows;
          } else {
            row0 = c * 128;
            owner = row0 / dist.seg_rows;
          }
          if (mode != 4 && owner == dist.rank) continue;           // own chunks are read where they are
          // a chunk is dealt out in STAGE_PARTS pieces of 16 rows to consecutive CTAs: with whole chunks per CTA a gather of a few
          // dozen chunks kept only that many SMs copying (one issuing thread each) while the tiles of all SMs waited for them
          // (token dispatch keeps whole chunks: it has hundreds of them, and 16-row pieces cost it more in per-piece drains and
          // lock-step chunk completion than they gain)
          const int n_parts = mode == 4 ? 1 : STAGE_PARTS;
          const int PART_ROWS = 128 / n_parts;
          for (int part = 0; part < n_parts && ok; ++part) {
          if ((mine++ % gridDim.x) != blockIdx.x) continue;
          const int r_lo = part * PART_ROWS;
          const int n_items = max(0, min(PART_ROWS, rows - r_lo)) * nseg;
          for (int base = 0; base < n_items && ok; base += DISPATCH_SLOTS) {
            // the stores of the previous batch must have read their slots before new rows land there
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            const int nb = min(DISPATCH_SLOTS, n_items - base);
            // token dispatch: the batch's row-table entries are fetched together before any copy is issued (each copy's
            // asm statement orders memory, so entries read one by one inside the loop would cost one global-load latency per row)
            int ent[DISPATCH_SLOTS];
            if (mode == 4) {
#pragma unroll
              for (int j = 0; j < DISPATCH_SLOTS; ++j) ent[j] = j < nb ? __ldg(dist.row_src + row0 + r_lo + (base + j) / nseg) : -1;
            }
            for (int j = 0; j < nb; ++j) {
              const int it = base + j, r = r_lo + it / nseg, sg = it - (it / nseg) * nseg;
              const int off = sg * DISPATCH_SLOT_BYTES;
              const uint32_t bytes = (uint32_t)min(DISPATCH_SLOT_BYTES, row_bytes - off);
              const bf16* src = nullptr;
              if (mode == 4) {
                const int e = ent[j];
                if (e >= 0) src = srcs[e >> 24] + (long)(e & 0xFFFFFF) * dist.ld_seg;
              } else if (by_k) {
                src = srcs[owner] + (long)(dist.row_off + row0 + r) * dist.ld_seg;
              } else {
                src = srcs[owner] + (long)(row0 + r - owner * dist.seg_rows) * dist.ld_seg;
              }
              if (src != nullptr) {
                mbar_expect_tx(&bbar[j], bytes);
                bulk_load_1d(bounce + j * DISPATCH_SLOT_BYTES, reinterpret_cast<const uint8_t*>(src) + off, bytes, &bbar[j]);
              } else {
                mbar_arrive(&bbar[j]);                            // padding row: keeps the slot's phase in step with the others
              }
            }
            for (int j = 0; j < nb; ++j) {
              const int it = base + j, r = r_lo + it / nseg, sg = it - (it / nseg) * nseg;
              const int off = sg * DISPATCH_SLOT_BYTES;
              const uint32_t bytes = (uint32_t)min(DISPATCH_SLOT_BYTES, row_bytes - off);
              const bool pad = mode == 4 && ent[j] < 0;
              if (!mbar_wait(&bbar[j], phase, abort_flag, err_word, VB_ERR_WAIT_FULL)) { ok = false; break; }
              uint8_t* dst = reinterpret_cast<uint8_t*>(stage + (long)(row0 + r) * dist.ld_stage + dst_col) + off;
              bulk_store_1d(dst, pad ? zero_row : bounce + j * DISPATCH_SLOT_BYTES, bytes);
            }
            for (int j = nb; j < DISPATCH_SLOTS; ++j) mbar_arrive(&bbar[j]);        // unused slots of a short last batch
            tma_store_commit();
            phase ^= 1;
          }
          tma_store_wait_all();                                   // this piece's rows are in the staging buffer
          asm volatile("fence.proxy.async;" ::: "memory");
          // the launcher zeroes the flags of the call's chunks; a chunk is complete when all its pieces have reported
          asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(dist.stage_flags + c), "r"(STAGE_PARTS / n_parts) : "memory");
          }
        }
        tma_store_wait_all();
      }
    }
    }
  } else {
    // ------------------------------------------------------------ epilogue (128 threads)
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const bool out_f32 = flags & GEMM_OUT_F32;
    const bool accum = flags & GEMM_ACCUM;
    uint32_t it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
      int mb, nb;
      long c_off = 0;                                  // element offset of this tile's output matrix inside Cv
      if (dist.group_mode == 2) {
        const int expert = t / (num_m * num_n);
        tile_coords(t - expert * num_m * num_n, mb, nb);
        const int2 rng = dist.expert_rng[expert];
        if (rng.y <= rng.x) { --it; continue; }
        c_off = (long)expert * M * ldc;
      } else {
        tile_coords(t, mb, nb);
        if (dist.group_mode == 1 && dist.blk_expert[mb] < 0) { --it; continue; }
      }
      const uint32_t acc = it & 1;
      const uint32_t acc_ph = (it >> 1) & 1;
      if (!mbar_wait(&tfull_bar[acc], acc_ph, abort_flag, err_word, VB_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int row = mb * BM + q * 32 + lane;
      const int n0 = nb * BN;
      const uint32_t taddr = tmem_base + acc * BN + (uint32_t(q * 32) << 16);
      if constexpr (EPI == EPI_LOGPROB) {
        // online softmax statistics of this row over the BN columns of the tile; one thread owns one row
        float m_run = -INFINITY, s_run = 0.f, sx_run = 0.f;
        const long label = (row < M) ? epi.labels[row] - epi.col_offset : -1;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(taddr + c * 32, v);
          tmem_ld_wait();
          const int col0 = n0 + c * 32;
          float x[32];
          float cmax = -INFINITY;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            x[j] = (col0 + j < N) ? __uint_as_float(v[j]) * epi.inv_temp : -INFINITY;
            cmax = fmaxf(cmax, x[j]);
          }
          if (cmax > -INFINITY) {
            const float m_new = fmaxf(m_run, cmax);
            const float a = __expf(m_run - m_new);
            float cs = 0.f, cx = 0.f;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float e = __expf(x[j] - m_new);
              cs += e;
              cx += (col0 + j < N) ? e * x[j] : 0.f;
            }
            s_run = s_run * a + cs;
            sx_run = sx_run * a + cx;
            m_run = m_new;
          }
          if (label >= col0 && label < col0 + 32 && label < N && row < M) {   // a label in the padding of the last tile is out of range
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (label == col0 + j) epi.label_logit[row] = x[j];
          }
        }
        if (row < M) {
          const long pi = (long)nb * M + row;
          epi.part_max[pi] = m_run;
          epi.part_sum[pi] = s_run;
          epi.part_sumx[pi] = sx_run;
        }
      } else if constexpr (EPI == EPI_DLOGITS) {
        float lse = 0.f, hh = 0.f, glp = 0.f, gen = 0.f;
        long label = -1;
        if (row < M) {
          lse = epi.lse[row];
          glp = epi.g_lp[row];
          if (epi.g_ent != nullptr) { gen = epi.g_ent[row]; hh = epi.ent[row]; }
          label = epi.labels[row] - epi.col_offset;
        }
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(taddr + c * 32, v);
          tmem_ld_wait();
          const int col0 = n0 + c * 32;
          if (row < M && col0 < N) {
            float f[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float x = __uint_as_float(v[j]) * epi.inv_temp;
              const float pr = __expf(x - lse);
              float g = -glp * pr - gen * pr * (x - lse + hh);
              if (label == col0 + j) g += glp;
              f[j] = g * epi.inv_temp;
            }
            bf16* crow = reinterpret_cast<bf16*>(Cv) + (size_t)row * ldc + col0;
            if (col0 + 32 <= N && ((reinterpret_cast<uintptr_t>(crow) & 15) == 0)) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 o;
                o.x = pack_bf16x2(f[j], f[j + 1]);
                o.y = pack_bf16x2(f[j + 2], f[j + 3]);
                o.z = pack_bf16x2(f[j + 4], f[j + 5]);
                o.w = pack_bf16x2(f[j + 6], f[j + 7]);
                *reinterpret_cast<uint4*>(crow + j) = o;
              }
            } else {
              for (int j = 0; j < 32; ++j)
                if (col0 + j < N) crow[j] = __float2bfloat16(f[j]);
            }
          }
        }
      } else if constexpr (EPI == EPI_PEER) {
        if (dist.row_dst != nullptr) {
          // Expert outputs go straight to the rank and row of the token they belong to, scaled by the routing weight. A thread
          // owns one output row; it packs 64 columns into its own 128-byte line of shared memory (line pitch 144 B: the eight
          // lanes of a 16-byte store phase hit eight different bank groups) and sends the line as ONE bulk store, so a row
          // crosses NVLink in 128-byte writes from the copy engine instead of 64-byte stores from the thread.
          const int e = row < M ? dist.row_dst[row] : -1;
          const float w = e >= 0 ? dist.row_w[row] : 0.f;
          bf16* drow = e >= 0 ? reinterpret_cast<bf16*>(dist.peer_out[e >> 24]) + (long)(e & 0xFFFFFF) * ldc : nullptr;
          uint8_t* line = smem + STAGES * Cfg::STAGE_BYTES + 256 + (q * 32 + lane) * COMBINE_LINE_PITCH;
#pragma unroll 1
          for (int c = 0; c < BN / 64; ++c) {
            uint32_t v[64];
            tmem_ld_32x32b_x32(taddr + c * 64, v);
            tmem_ld_32x32b_x32(taddr + c * 64 + 32, v + 32);
            tmem_ld_wait();
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");      // the previous store has read this line
            const int col0 = n0 + c * 64;
            if (e >= 0 && col0 + 64 <= N) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                uint4 o;
                o.x = pack_bf16x2(__uint_as_float(v[8 * j]) * w, __uint_as_float(v[8 * j + 1]) * w);
                o.y = pack_bf16x2(__uint_as_float(v[8 * j + 2]) * w, __uint_as_float(v[8 * j + 3]) * w);
                o.z = pack_bf16x2(__uint_as_float(v[8 * j + 4]) * w, __uint_as_float(v[8 * j + 5]) * w);
                o.w = pack_bf16x2(__uint_as_float(v[8 * j + 6]) * w, __uint_as_float(v[8 * j + 7]) * w);
                reinterpret_cast<uint4*>(line)[j] = o;
              }
              fence_async_smem();                                                 // the line was written by ordinary stores
              bulk_store_1d(drow + col0, line, 128);
              tma_store_commit();
            }
          }
          tc_fence_before();
          mbar_arrive(&tempty_bar[acc]);
          continue;
        }
        int r_lo = 0, r_hi = dist.world;
        long row_local = row;
        if (dist.sig_local != nullptr) {          // signalled all-reduce: partials stay local, the peers pull them
          r_lo = dist.rank;
          r_hi = r_lo + 1;
        } else if (dist.rows_per_owner > 0) {
          r_lo = row / dist.rows_per_owner;
          r_hi = r_lo + 1;
          row_local = row - (long)r_lo * dist.rows_per_owner;
        }
        if (dist.peer_lines) {
          // 64 output columns of this thread's row are packed into its shared-memory line and leave as one 128-byte bulk store
          // per destination (see the combine epilogue above): the copy engine writes to the peers, not the thread
          uint8_t* line = smem + STAGES * Cfg::STAGE_BYTES + 256 + (q * 32 + lane) * COMBINE_LINE_PITCH;
#pragma unroll 1
          for (int c = 0; c < BN / 64; ++c) {
            uint32_t v[64];
            tmem_ld_32x32b_x32(taddr + c * 64, v);
            tmem_ld_32x32b_x32(taddr + c * 64 + 32, v + 32);
            tmem_ld_wait();
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");      // the previous store has read this line
            const int col0 = n0 + c * 64;
            if (row < M && col0 + 64 <= N) {
              if (bias != nullptr) {
#pragma unroll
                for (int j = 0; j < 64; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + __bfloat162float(bias[col0 + j]));
              }
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                uint4 o;
                o.x = pack_bf16x2(__uint_as_float(v[8 * j]), __uint_as_float(v[8 * j + 1]));
                o.y = pack_bf16x2(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]));
                o.z = pack_bf16x2(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]));
                o.w = pack_bf16x2(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]));
                reinterpret_cast<uint4*>(line)[j] = o;
              }
              fence_async_smem();
              if (dist.head_dim > 0) {
                const uint16_t e = dist.head_map[col0 / dist.head_dim];
                bf16* dst = reinterpret_cast<bf16*>(dist.peer_out[e >> 12]) + ((long)dist.row_off + row) * ldc +
                            (long)(e & 0xFFF) * dist.head_dim + (col0 % dist.head_dim);
                bulk_store_1d(dst, line, 128);
              } else {
                for (int r = r_lo; r < r_hi; ++r) {
                  const long slot = dist.sig_local != nullptr ? (long)(t % split_k) : (long)dist.rank;
                  bf16* dst = reinterpret_cast<bf16*>(dist.peer_out[r]) + sig_slot_off + slot * dist.slot_elems + row_local * ldc + col0;
                  bulk_store_1d(dst, line, 128);
                }
              }
              tma_store_commit();
            }
          }
          tc_fence_before();
          mbar_arrive(&tempty_bar[acc]);
          continue;
        }
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(taddr + c * 32, v);
          tmem_ld_wait();
          const int col0 = n0 + c * 32;
          if (row < M && col0 + 32 <= N) {
            if (bias != nullptr) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + __bfloat162float(bias[col0 + j]));
            }
            uint4 o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              o[j].x = pack_bf16x2(__uint_as_float(v[8 * j]), __uint_as_float(v[8 * j + 1]));
              o[j].y = pack_bf16x2(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]));
              o[j].z = pack_bf16x2(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]));
              o[j].w = pack_bf16x2(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]));
            }
            if (dist.head_dim > 0) {
              // all-to-all by heads: this rank's token rows land at row_off + row of the head owner's [T, local heads] buffer
              const uint16_t e = dist.head_map[col0 / dist.head_dim];
              bf16* dst = reinterpret_cast<bf16*>(dist.peer_out[e >> 12]) + ((long)dist.row_off + row) * ldc +
                          (long)(e & 0xFFF) * dist.head_dim + (col0 % dist.head_dim);
#pragma unroll
              for (int j = 0; j < 4; ++j) reinterpret_cast<uint4*>(dst)[j] = o[j];
              continue;
            }
            for (int r = r_lo; r < r_hi; ++r) {
              const long slot = dist.sig_local != nullptr ? (long)(t % split_k) : (long)dist.rank;
              bf16* dst = reinterpret_cast<bf16*>(dist.peer_out[r]) + sig_slot_off + slot * dist.slot_elems + row_local * ldc + col0;
#pragma unroll
              for (int j = 0; j < 4; ++j) reinterpret_cast<uint4*>(dst)[j] = o[j];
            }
          }
        }
      } else {
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(taddr + c * 32, v);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        if (row < M && col0 < N) {
          float f[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
          if (split_k > 1) {
            // partial sum of this K slice: fp32 workspace [split][M][N]; bias / accumulate / cast happen in the reduce pass
            float* wrow = split_ws + ((size_t)(t % split_k) * M + row) * N + col0;
            if (col0 + 32 <= N && ((reinterpret_cast<uintptr_t>(wrow) & 15) == 0)) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(wrow + j) = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
            } else {
              for (int j = 0; j < 32; ++j)
                if (col0 + j < N) wrow[j] = f[j];
            }
            continue;
          }
          if (bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < N) f[j] += __bfloat162float(bias[col0 + j]);
          }
          const bool full = (col0 + 32 <= N);
          if (out_f32) {
            float* crow = reinterpret_cast<float*>(Cv) + c_off + (size_t)row * ldc + col0;
            if (full && ((reinterpret_cast<uintptr_t>(crow) & 15) == 0)) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                float4 o = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
                if (accum) {
                  float4 p = *reinterpret_cast<float4*>(crow + j);
                  o.x += p.x; o.y += p.y; o.z += p.z; o.w += p.w;
                }
                *reinterpret_cast<float4*>(crow + j) = o;
              }
            } else {
              for (int j = 0; j < 32; ++j)
                if (col0 + j < N) crow[j] = accum ? crow[j] + f[j] : f[j];
            }
          } else {
            bf16* crow = reinterpret_cast<bf16*>(Cv) + c_off + (size_t)row * ldc + col0;
            if (full && ((reinterpret_cast<uintptr_t>(crow) & 15) == 0)) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                if (accum) {
                  uint4 p = *reinterpret_cast<uint4*>(crow + j);
                  const __nv_bfloat162* ph2 = reinterpret_cast<const __nv_bfloat162*>(&p);
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    float2 pf = __bfloat1622float2(ph2[e]);
                    f[j + 2 * e] += pf.x;
                    f[j + 2 * e + 1] += pf.y;
                  }
                }
                uint4 o;
                o.x = pack_bf16x2(f[j], f[j + 1]);
                o.y = pack_bf16x2(f[j + 2], f[j + 3]);
                o.z = pack_bf16x2(f[j + 4], f[j + 5]);
                o.w = pack_bf16x2(f[j + 6], f[j + 7]);
                *reinterpret_cast<uint4*>(crow + j) = o;
              }
            } else {
              for (int j = 0; j < 32; ++j)
                if (col0 + j < N) {
                  float o = accum ? __bfloat162float(crow[j]) + f[j] : f[j];
                  crow[j] = __float2bfloat16(o);
                }
            }
          }
        }
      }
      }
      tc_fence_before();
      mbar_arrive(&tempty_bar[acc]);
    }
    if (EPI == EPI_PEER && (dist.row_dst != nullptr || dist.peer_lines)) tma_store_wait_all();   // this thread's bulk stores have landed
  }

  // ------------------------------------------------------------ teardown
  if (EPI == EPI_PEER && dist.sig_local != nullptr) __threadfence_system();   // this thread's partials visible to the peers before the signal
  tc_fence_before();
  __syncthreads();
  if (EPI == EPI_PEER && dist.sig_local != nullptr && threadIdx.x == 0) {
    const int done = atomicAdd(dist.sig_local + 1, 1);
    if (done == (int)gridDim.x - 1) {                 // every CTA of this launch has published its tiles
      dist.sig_local[1] = 0;
      const int e = dist.sig_local[0] + 1;
      dist.sig_local[0] = e;
      __threadfence_system();
      for (int p = 0; p < dist.world; ++p)
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(dist.sig_peer[p] + SIG_FLAGS + dist.rank), "r"(e) : "memory");
    }
  }
  if (warp == 1) {
    if (*abort_flag) {
      // A wait was abandoned: give copies and MMAs still in flight time to land before TMEM and the
      // shared-memory ring go away with the CTA.
      uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 2000000ull) { __nanosleep(1000); }
    }
    tc_fence_after();
    tmem_dealloc<Cfg::TMEM_COLS>(tmem_base);
  }
}

// ---------------------------------------------------------------- split-K reduce
// out[m,n] (+)= sum_s ws[s,m,n] (+ bias[n]); out is bf16 or fp32 with row stride ldc.
__global__ void splitk_reduce_kernel(const float* __restrict__ ws, int S, int M, int N, void* __restrict__ out, int ldc,
                                     const bf16* __restrict__ bias, int flags) {
  const long total4 = (long)M * N / 4;
  const bool out_f32 = flags & GEMM_OUT_F32, accum = flags & GEMM_ACCUM;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total4; i += (long)gridDim.x * blockDim.x) {
    const long e = i * 4;
    const int row = e / N, col = e % N;
    float4 a = reinterpret_cast<const float4*>(ws)[i];
    for (int s2 = 1; s2 < S; ++s2) {
      const float4 b = reinterpret_cast<const float4*>(ws + (size_t)s2 * M * N)[i];
      a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
    }
    if (bias != nullptr) {
      a.x += __bfloat162float(bias[col]); a.y += __bfloat162float(bias[col + 1]);
      a.z += __bfloat162float(bias[col + 2]); a.w += __bfloat162float(bias[col + 3]);
    }
    if (out_f32) {
      float* o = reinterpret_cast<float*>(out) + (size_t)row * ldc + col;
      if (accum) { a.x += o[0]; a.y += o[1]; a.z += o[2]; a.w += o[3]; }
      o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w;
    } else {
      bf16* o = reinterpret_cast<bf16*>(out) + (size_t)row * ldc + col;
      if (accum) {
        a.x += __bfloat162float(o[0]); a.y += __bfloat162float(o[1]); a.z += __bfloat162float(o[2]); a.w += __bfloat162float(o[3]);
      }
      o[0] = __float2bfloat16(a.x); o[1] = __float2bfloat16(a.y); o[2] = __float2bfloat16(a.z); o[3] = __float2bfloat16(a.w);
    }
  }
}

// ---------------------------------------------------------------- host launcher
static int g_num_sms = 0;

static int num_sms() {
  if (g_num_sms == 0) {
    int dev;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return g_num_sms;
}

template <int BN, bool A_MN, bool B_MN, int EPI = EPI_STORE, int COPY_WARPS = 0, int KA = 1>
static int launch_gemm(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda, int ldb,
                       int ldc, int flags, int* err_word, cudaStream_t stream, const LmHeadEpi& epi = LmHeadEpi{},
                       int split_k = 1, float* split_ws = nullptr, const DistArgs* dist_in = nullptr) {
  using Cfg = GemmCfg<BN, KA>;
  static const DistArgs no_dist = {};
  DistArgs dist = dist_in ? *dist_in : no_dist;
  if (EPI == EPI_PEER && dist.row_dst == nullptr)
    dist.peer_lines = (N % 64 == 0) && (dist.head_dim == 0 || dist.head_dim % 64 == 0) && (ldc % 8 == 0) && (dist.slot_elems % 8 == 0) &&
                      (dist.sig_half % 8 == 0);
  CUtensorMap tmA, tmB;
  int rc;
  if (!A_MN) rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, BM, BK);
  else       rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, lda, BK, 64);
  if (rc) return rc;
  if (!B_MN) rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldb, BN, BK);
  else       rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, ldb, BK, 64);
  if (rc) return rc;
  // kernels with staging warps carry the bulk-copy ring behind the pipeline stages
  constexpr int SMEM = Cfg::SMEM_BYTES + (COPY_WARPS > 0 ? DISPATCH_SMEM_BYTES : 0) + (EPI == EPI_PEER ? COMBINE_SMEM_BYTES : 0);
  static_assert(SMEM <= 227 * 1024, "pipeline stages + staging ring exceed the shared memory of an SM");
  static bool attr_set = false;
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, EPI, COPY_WARPS, KA>;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return -10;
    attr_set = true;
  }
  const int num_kb = (K + BK * KA - 1) / (BK * KA);
  if (split_k < 1) split_k = 1;
  int kb_per = (num_kb + split_k - 1) / split_k;
  split_k = (num_kb + kb_per - 1) / kb_per;          // no empty slices
  if (split_k > 1 && split_ws == nullptr && EPI != EPI_PEER) return -6;
  int units = ((M + BM - 1) / BM) * ((N + BN - 1) / BN) * split_k;
  int grid = units < num_sms() ? units : num_sms();
  kern<<<grid, 192 + 32 * COPY_WARPS, SMEM, stream>>>(tmA, tmB, C, reinterpret_cast<const bf16*>(bias), M, N, K, ldc, flags,
                                                err_word, epi, split_k, kb_per, split_ws, dist);
  if (cudaGetLastError() != cudaSuccess) return -11;
  if (split_k > 1 && EPI != EPI_PEER) {
    long total4 = (long)M * N / 4;
    int blocks = (int)((total4 + 255) / 256);
    if (blocks > num_sms() * 8) blocks = num_sms() * 8;
    splitk_reduce_kernel<<<blocks, 256, 0, stream>>>(split_ws, split_k, M, N, C, ldc, reinterpret_cast<const bf16*>(bias), flags);
    if (cudaGetLastError() != cudaSuccess) return -12;
  }
  return 0;
}

}  // namespace vb

// out[M,N] (+)= sum over S fp32 partials ws[s][M][N] (+ bias): the reduce pass of the split-K GEMMs, also used by the paired-CTA kernel.
extern "C" int vb_splitk_reduce(const float* ws, int S, int M, int N, void* out, int ldc, const void* bias, int out_f32, int accumulate,
                                cudaStream_t stream) {
  using namespace vb;
  if ((long)M * N % 4) return -2;
  const long total4 = (long)M * N / 4;
  int blocks = (int)((total4 + 255) / 256);
  if (blocks > num_sms() * 8) blocks = num_sms() * 8;
  const int flags = (out_f32 ? GEMM_OUT_F32 : 0) | (accumulate ? GEMM_ACCUM : 0);
  splitk_reduce_kernel<<<blocks, 256, 0, stream>>>(ws, S, M, N, out, ldc, reinterpret_cast<const bf16*>(bias), flags);
  return cudaGetLastError() == cudaSuccess ? 0 : -12;
}

namespace vb {

// Cost model for small problems that cannot fill the machine with 128x256 tiles: pick (tile width, K splits) minimising
// waves x (bytes staged per unit / per-SM fill rate + fixed cost) + the reduce pass.
static void pick_tile_and_split(int M, int N, int K, bool b_mn, int* bn_out, int* split_out) {
  const int sms = num_sms();
  const int num_m = (M + BM - 1) / BM;
  const int num_kb = (K + BK - 1) / BK;
  double best = 1e30;
  int best_bn = 256, best_s = 1;
  const int bns[4] = {256, 128, 64, 32};
  for (int bi = 0; bi < 4; ++bi) {
    const int bn = bns[bi];
    if (b_mn && bn < 64) continue;
    const long tiles = (long)num_m * ((N + bn - 1) / bn);
    for (int s = 1; s <= 16; ++s) {
      if (s > 1 && (N % 4 != 0)) break;                 // the reduce pass is vectorised by 4 columns
      const int kb_per = (num_kb + s - 1) / s;
      if (s > 1 && kb_per < 4) break;
      const int s_eff = (num_kb + kb_per - 1) / kb_per;
      const long units = tiles * s_eff;
      const double waves = (double)((units + sms - 1) / sms);
      const double unit_us = kb_per * (double)(A_TILE_BYTES + bn * BK * 2) / 100e3 /* ~100 GB/s per SM */ + 2.5;
      double t = waves * unit_us;
      if (s_eff > 1) t += 3.0 + 2.0 * s_eff * (double)M * N * 4 / 5e6 /* ~5 TB/s */;
      if (t < best) { best = t; best_bn = bn; best_s = s_eff; }
      if (units >= 4L * sms) break;
    }
  }
  *bn_out = best_bn;
  *split_out = best_s;
}

}  // namespace vb

// C[M,N] (+)= op(A) op(B) (+ bias). a_mn / b_mn: 0 = K contiguous ([M,K] / [N,K] row-major), 1 = M/N contiguous
// ([K,M] / [K,N] row-major). lda/ldb/ldc are row strides in elements. Requirements: A, B 16-byte aligned,
// lda/ldb multiples of 8. `bn` = 0 picks the N tile from the problem shape.
extern "C" void vb_gemm_plan(int M, int N, int K, int b_mn, int bn_req, int* bn, int* split_k) {
  using namespace vb;
  *split_k = 1;
  if (bn_req != 0) {
    *bn = bn_req;
    return;
  }
  const long big_tiles = (long)((M + BM - 1) / BM) * ((N + 255) / 256);
  if (big_tiles >= num_sms()) { *bn = 256; return; }
  pick_tile_and_split(M, N, K, b_mn != 0, bn, split_k);
}

// split_k > 1 needs split_ws with split_k * M * N floats (see vb_gemm_plan); split_k = 1 ignores it.
extern "C" int vb_gemm_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda,
                            int ldb, int ldc, int a_mn, int b_mn, int out_f32, int accumulate, int bn, int split_k,
                            float* split_ws, int* err_word, cudaStream_t stream) {
  using namespace vb;
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return -3;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda & 7) || (ldb & 7)) return -4;
  int flags = (out_f32 ? GEMM_OUT_F32 : 0) | (accumulate ? GEMM_ACCUM : 0);
  if (bn == 0) {
    int s_auto;
    vb_gemm_plan(M, N, K, b_mn, 0, &bn, &s_auto);
    if (split_k == 0) split_k = s_auto;
  }
  if (split_k < 1) split_k = 1;
  if (split_k > 1 && (N % 4 != 0)) split_k = 1;
  if (b_mn && bn < 64) bn = 64;
#define VB_LAUNCH(BN_, AM_, BM_) \
  return launch_gemm<BN_, AM_, BM_>(A, B, C, bias, M, N, K, lda, ldb, ldc, flags, err_word, stream, LmHeadEpi{}, split_k, split_ws)
#define VB_DISPATCH_BN(AM_, BM_)                   \
  switch (bn) {                                    \
    case 256: VB_LAUNCH(256, AM_, BM_);            \
    case 128: VB_LAUNCH(128, AM_, BM_);            \
    case 64: VB_LAUNCH(64, AM_, BM_);              \
    default: break;                                \
  }
  if (!a_mn && !b_mn) {
    if (bn == 32) VB_LAUNCH(32, false, false);
    // decode-sized problems (at most four row blocks) are memory bound: 256-byte row bursts per stage (KA = 2)
    // (measured on B200, M=256: N=4608,K=3584 25.6 -> 23.6 us; with K slices the single-atom stages stay ahead)
    if (M <= 4 * BM && split_k == 1) {
      switch (bn) {
        case 256: return launch_gemm<256, false, false, EPI_STORE, 0, 2>(A, B, C, bias, M, N, K, lda, ldb, ldc, flags, err_word, stream, LmHeadEpi{}, split_k, split_ws);
        case 128: return launch_gemm<128, false, false, EPI_STORE, 0, 2>(A, B, C, bias, M, N, K, lda, ldb, ldc, flags, err_word, stream, LmHeadEpi{}, split_k, split_ws);
        case 64: return launch_gemm<64, false, false, EPI_STORE, 0, 2>(A, B, C, bias, M, N, K, lda, ldb, ldc, flags, err_word, stream, LmHeadEpi{}, split_k, split_ws);
        default: break;
      }
    }
    VB_DISPATCH_BN(false, false)
  } else if (!a_mn && b_mn) {
    VB_DISPATCH_BN(false, true)
  } else if (a_mn && b_mn) {
    VB_DISPATCH_BN(true, true)
  } else {
    VB_DISPATCH_BN(true, false)
  }
  return -5;
}

// ---------------------------------------------------------------------------------------------------------------
// Fused lm_head -> log-prob / entropy. Forward never writes logits: each 128x256 tile of h W^T leaves the SM as three
// partial softmax statistics per row; a second tiny kernel merges the partials.
// Replaces the reference's Triton kernels (verl/utils/kernel/kernels.py:186-563) and the torch-chunked
// FusedLinearForPPO (verl/utils/experimental/torch_functional.py:96-217).
namespace vb {

constexpr int LM_BN = 256;

__global__ void lmhead_merge_kernel(const float* __restrict__ pmax, const float* __restrict__ psum, const float* __restrict__ psumx,
                                    const float* __restrict__ label_logit, int M, int num_n, float* __restrict__ logp,
                                    float* __restrict__ ent, float* __restrict__ lse_out) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= M) return;
  float m = -INFINITY;
  for (int nb = 0; nb < num_n; ++nb) m = fmaxf(m, pmax[(long)nb * M + row]);
  float s = 0.f, sx = 0.f;
  for (int nb = 0; nb < num_n; ++nb) {
    const long i = (long)nb * M + row;
    const float pm = pmax[i];
    const float w = (pm == -INFINITY) ? 0.f : __expf(pm - m);
    s += w * psum[i];
    sx += w * psumx[i];
  }
  const float lse = m + logf(s);
  logp[row] = label_logit[row] - lse;
  if (ent != nullptr) ent[row] = lse - sx / s;
  if (lse_out != nullptr) lse_out[row] = lse;
}

}  // namespace vb

extern "C" long vb_lmhead_scratch_floats(int M, int V) {
  const long num_n = (V + vb::LM_BN - 1) / vb::LM_BN;
  return 3 * num_n * (long)M + M;
}

// h: [M, K] bf16 (row stride ldh), W: [V, K] bf16 (row stride ldw), labels: int64 [M].
// scratch: vb_lmhead_scratch_floats(M, V) floats. Outputs fp32 [M]: logp, ent (nullable), lse (nullable).
// A row whose label lies outside [0, V) gets logp = -lse.
extern "C" int vb_lmhead_logprob_fwd(const void* h, const void* W, const long* labels, int M, int V, int K, int ldh, int ldw,
                                     float inv_temp, float* scratch, float* logp, float* ent, float* lse, int* err_word,
                                     cudaStream_t stream) {
  using namespace vb;
  if (M <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(h) & 15) || (reinterpret_cast<uintptr_t>(W) & 15) || (ldh & 7) || (ldw & 7)) return -4;
  const long num_n = (V + LM_BN - 1) / LM_BN;
  LmHeadEpi epi = {};
  epi.inv_temp = inv_temp;
  epi.labels = labels;
  epi.col_offset = 0;
  epi.part_max = scratch;
  epi.part_sum = scratch + num_n * M;
  epi.part_sumx = scratch + 2 * num_n * M;
  epi.label_logit = scratch + 3 * num_n * M;
  // the label-logit section is only written for rows whose label is a column of W: rows with a label outside [0, V)
  // (ignore index, padded vocabulary) must read zero, not whatever the scratch held before
  if (cudaMemsetAsync(epi.label_logit, 0, sizeof(float) * (size_t)M, stream) != cudaSuccess) return -13;
  int rc = launch_gemm<LM_BN, false, false, EPI_LOGPROB>(h, W, nullptr, nullptr, M, V, K, ldh, ldw, 0, 0, err_word, stream, epi);
  if (rc) return rc;
  lmhead_merge_kernel<<<(M + 127) / 128, 128, 0, stream>>>(epi.part_max, epi.part_sum, epi.part_sumx, epi.label_logit, M,
                                                           (int)num_n, logp, ent, lse);
  return cudaGetLastError() == cudaSuccess ? 0 : -12;
}

// dlogits[M, Vc] (bf16, row stride ldd) for vocabulary columns [col_offset, col_offset + Vc): W points at row col_offset.
extern "C" int vb_lmhead_dlogits(const void* h, const void* W, const long* labels, int M, int Vc, int K, int ldh, int ldw,
                                 float inv_temp, int col_offset, const float* lse, const float* ent, const float* g_lp,
                                 const float* g_ent, void* dlogits, int ldd, int* err_word, cudaStream_t stream) {
  using namespace vb;
  if (M <= 0 || Vc <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(h) & 15) || (reinterpret_cast<uintptr_t>(W) & 15) || (ldh & 7) || (ldw & 7)) return -4;
  LmHeadEpi epi = {};
  epi.inv_temp = inv_temp;
  epi.labels = labels;
  epi.col_offset = col_offset;
  epi.lse = lse; epi.ent = ent; epi.g_lp = g_lp; epi.g_ent = g_ent;
  return launch_gemm<LM_BN, false, false, EPI_DLOGITS>(h, W, dlogits, nullptr, M, Vc, K, ldh, ldw, ldd, 0, err_word, stream, epi);
}

// ---------------------------------------------------------------------------------------------------------------
// GEMMs fused with tensor/data-parallel collectives over NVLink peer memory.
namespace vb {

// Slot sum of the signalled all-reduce (one-shot, pull): every block first waits (bounded) until all ranks' flags have
// reached this rank's epoch, then reads every rank's K-slice partials straight from that rank's memory (coalesced 16-byte
// loads over NVLink) and sums them in fp32. The buffer half is selected by the epoch's parity.
struct PeerSlots {
  const bf16* p[MAX_TP];
};

__global__ void slots_reduce_sig_kernel(const __grid_constant__ PeerSlots peers, const int* __restrict__ sig, int rank, int world, int split_k, long slot_elems,
                                        long half_elems, long rows, int cols, const bf16* __restrict__ residual, bf16* __restrict__ out,
                                        int ld_out, int* err_word) {
  __shared__ int ok_s;
  const int e = sig[0];
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (threadIdx.x < world) {
    const int* f = sig + SIG_FLAGS + threadIdx.x;
    uint64_t t0 = 0;
    uint32_t n = 0;
    while (true) {
      int v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
      if (v >= e) break;
      if ((++n & 0xFF) == 0) {
        const uint64_t now = globaltimer_ns();
        if (t0 == 0) t0 = now;
        if (now - t0 > VB_WAIT_LIMIT_NS) {
          atomicCAS(err_word, 0, VB_ERR_WAIT_PEER | (threadIdx.x << 8));
          ok_s = 0;
          break;
        }
        __nanosleep(100);
      }
    }
  }
  __syncthreads();
  if (!ok_s) return;
  const long base = (long)((e - 1) & 1) * half_elems;
  const int vpr = cols / 8;
  const long total = rows * vpr;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long r = i / vpr;
    const int c = (i % vpr) * 8;
    const long off = base + r * cols + c;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int q = 0; q < world; ++q) {
      const bf16* src = peers.p[(rank + q) % world] + off;        // own partial first while the remote loads are in flight
      for (int s2 = 0; s2 < split_k; ++s2) {
        const uint4 v = *reinterpret_cast<const uint4*>(src + s2 * slot_elems);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f2 = __bfloat1622float2(h[k]);
          acc[2 * k] += f2.x;
          acc[2 * k + 1] += f2.y;
        }
      }
    }
    if (residual != nullptr) {
      const uint4 v = *reinterpret_cast<const uint4*>(residual + r * ld_out + c);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f2 = __bfloat1622float2(h[k]);
        acc[2 * k] += f2.x;
        acc[2 * k + 1] += f2.y;
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + r * ld_out + c) = o;
  }
}

// out[r, c] = sum_s slots[s][r, c] (+ residual[r, c]); bf16 in/out, fp32 accumulation. cols % 8 == 0.
__global__ void slots_reduce_kernel(const bf16* __restrict__ slots, int world, long slot_elems, long rows, int cols, int ld,
                                    const bf16* __restrict__ residual, bf16* __restrict__ out, int ld_out) {
  const int vpr = cols / 8;
  const long total = rows * vpr;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long r = i / vpr;
    const int c = (i % vpr) * 8;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int s = 0; s < world; ++s) {
      const uint4 v = *reinterpret_cast<const uint4*>(slots + s * slot_elems + r * ld + c);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        acc[2 * e] += f.x;
        acc[2 * e + 1] += f.y;
      }
    }
    if (residual != nullptr) {
      const uint4 v = *reinterpret_cast<const uint4*>(residual + r * ld_out + c);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        acc[2 * e] += f.x;
        acc[2 * e + 1] += f.y;
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + r * ld_out + c) = o;
  }
}

template <int EPI, bool B_MN = false>
static int launch_dist(int bn, const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda, int ldb, int ldc,
                       int* err_word, cudaStream_t st, const DistArgs& d, int split_k = 1) {
  if constexpr (EPI == EPI_STORE) {
    if (d.stage != nullptr) {
      switch (bn) {
        case 256: return launch_gemm<256, false, B_MN, EPI, 8>(A, B, C, bias, M, N, K, lda, ldb, ldc, 0, err_word, st, LmHeadEpi{}, 1, nullptr, &d);
        case 128: return launch_gemm<128, false, B_MN, EPI, 8>(A, B, C, bias, M, N, K, lda, ldb, ldc, 0, err_word, st, LmHeadEpi{}, 1, nullptr, &d);
        case 64: return launch_gemm<64, false, B_MN, EPI, 8>(A, B, C, bias, M, N, K, lda, ldb, ldc, 0, err_word, st, LmHeadEpi{}, 1, nullptr, &d);
        default: return -5;
      }
    }
  }
  if (EPI != EPI_PEER) split_k = 1;
  switch (bn) {
    case 256: return launch_gemm<256, false, B_MN, EPI>(A, B, C, bias, M, N, K, lda, ldb, ldc, 0, err_word, st, LmHeadEpi{}, split_k, nullptr, &d);
    case 128: return launch_gemm<128, false, B_MN, EPI>(A, B, C, bias, M, N, K, lda, ldb, ldc, 0, err_word, st, LmHeadEpi{}, split_k, nullptr, &d);
    case 64: return launch_gemm<64, false, B_MN, EPI>(A, B, C, bias, M, N, K, lda, ldb, ldc, 0, err_word, st, LmHeadEpi{}, split_k, nullptr, &d);
    default: return -5;
  }
}

static int pick_bn_dist(int M, int N) {
  int bn = 256;
  const int num_m = (M + BM - 1) / BM;
  while (bn > 64 && (long)num_m * ((N + bn - 1) / bn) < num_sms()) bn >>= 1;
  return bn;
}

}  // namespace vb

// All-gather fused into the GEMM: C[M,N] = A B^T (+bias) where the rows of A (which = 0) or of B (which = 1) are split in
// `world` equal segments; seg_ptrs[r] is rank r's segment ([seg_rows, K] bf16, row stride ld_seg) reachable from this GPU.
extern "C" int vb_gemm_allgather(int which, const long* seg_ptrs, int world, int seg_rows, int ld_seg, const void* other, int ld_other,
                                 void* C, const void* bias, int M, int N, int K, int ldc, int rank, void* stage, int* stage_flags,
                                 int stage_epoch, int b_mn, int* err_word, cudaStream_t st) {
  using namespace vb;
  if (world > MAX_TP || world < 1) return -2;
  if (b_mn && which != 0) return -2;             // the transposed form ([K, N] row-major) exists for the plain operand only
  const int rows_total = which == 0 ? M : N;
  if (seg_rows * world != rows_total || (ld_seg & 7) || (ld_other & 7)) return -4;
  const int bn = pick_bn_dist(M, N);
  const int tile_rows = which == 0 ? BM : bn;
  if (seg_rows % tile_rows != 0) return -6;      // a tile must not straddle two ranks' segments
  DistArgs d = {};
  d.seg_mode = which == 0 ? 1 : 2;
  d.seg_rows = seg_rows;
  d.n_seg = world;
  for (int r = 0; r < world; ++r) {
    if (make_tmap_2d(&d.seg[r], reinterpret_cast<const void*>(seg_ptrs[r]), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, seg_rows, K, ld_seg, tile_rows, BK))
      return -1;
  }
  if (stage != nullptr) {
    // `stage` is a local [rows_total, K] bf16 buffer (row stride K), `stage_flags` one int per 128 rows
    if (seg_rows % 128 != 0 || rank < 0 || rank >= world) return -6;
    d.stage = stage; d.stage_flags = stage_flags; d.stage_epoch = stage_epoch; d.ld_stage = K; d.ld_seg = ld_seg; d.rank = rank;
    for (int r = 0; r < world; ++r) d.seg_ptr[r] = reinterpret_cast<const void*>(seg_ptrs[r]);
    if (make_tmap_2d(&d.stage_map, stage, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows_total, K, K, tile_rows, BK)) return -1;
    // every 16-row piece of a chunk adds one to the chunk's flag: start the call from zero
    if (cudaMemsetAsync(stage_flags, 0, sizeof(int) * (rows_total / 128), st) != cudaSuccess) return -13;
  }
  const void* A = which == 0 ? reinterpret_cast<const void*>(seg_ptrs[0]) : other;
  const void* B = which == 0 ? other : reinterpret_cast<const void*>(seg_ptrs[0]);
  const int lda = which == 0 ? ld_seg : ld_other, ldb = which == 0 ? ld_other : ld_seg;
  // the unsegmented maps built by the launcher for the segmented operand are never used; give them legal extents
  const int Mm = which == 0 ? seg_rows : M, Nn = which == 1 ? seg_rows : N;
  (void)Mm; (void)Nn;
  if (b_mn) return launch_dist<EPI_STORE, true>(bn, A, B, C, bias, M, N, K, lda, ldb, ldc, err_word, st, d);
  return launch_dist<EPI_STORE>(bn, A, B, C, bias, M, N, K, lda, ldb, ldc, err_word, st, d);
}

// GEMM whose epilogue scatters the bf16 result into peers' symmetric slot buffers (see DistArgs). rows_per_owner == 0:
// every rank receives the whole [M,N] partial (all-reduce); > 0: only the owner of each row block (reduce-scatter).
extern "C" int vb_gemm_peer_scatter(const void* A, const void* B, int M, int N, int K, int lda, int ldb, int ld_slot,
                                    const long* out_ptrs, int rank, int world, int rows_per_owner, long slot_elems, int b_mn,
                                    int* err_word, cudaStream_t st) {
  using namespace vb;
  if (world > MAX_TP || (N % 32) != 0 || (ld_slot & 7)) return -2;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda & 7) || (ldb & 7)) return -4;
  DistArgs d = {};
  d.rank = rank; d.world = world; d.rows_per_owner = rows_per_owner; d.slot_elems = slot_elems;
  for (int r = 0; r < world; ++r) d.peer_out[r] = reinterpret_cast<void*>(out_ptrs[r]);
  if (b_mn) return launch_dist<EPI_PEER, true>(pick_bn_dist(M, N), A, B, nullptr, nullptr, M, N, K, lda, ldb, ld_slot, err_word, st, d);
  return launch_dist<EPI_PEER>(pick_bn_dist(M, N), A, B, nullptr, nullptr, M, N, K, lda, ldb, ld_slot, err_word, st, d);
}

// ---------------------------------------------------------------------------------------------------------------
// Grouped GEMMs of a mixture-of-experts layer (see DistArgs::group_mode). R = padded number of token rows.
namespace vb {
template <bool B_MN>
static int launch_grouped_fwd(const void* A, const void* B, void* C, const int* blk_expert, int R, int N, int K, int E, int lda, int ldc,
                              int* err_word, cudaStream_t stream) {
  constexpr int BN = 256;
  using Cfg = GemmCfg<BN>;
  CUtensorMap tmA, tmB;
  if (make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, R, K, lda, BM, BK)) return -1;
  int rc;
  if (!B_MN) rc = make_tmap_3d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, E, (uint64_t)K * 2, (uint64_t)N * K * 2, BK, BN, 1);
  else       rc = make_tmap_3d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, E, (uint64_t)N * 2, (uint64_t)N * K * 2, 64, BK, 1);
  if (rc) return rc;
  static bool attr_set = false;
  auto kern = gemm_bf16_kernel<BN, false, B_MN, EPI_STORE>;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess) return -10;
    attr_set = true;
  }
  DistArgs d = {};
  d.group_mode = 1; d.num_experts = E; d.blk_expert = blk_expert;
  const int units = (R / BM) * ((N + BN - 1) / BN);
  const int grid = units < num_sms() ? units : num_sms();
  const int num_kb = (K + BK - 1) / BK;
  kern<<<grid, 192, Cfg::SMEM_BYTES, stream>>>(tmA, tmB, C, nullptr, R, N, K, ldc, 0, err_word, LmHeadEpi{}, 1, num_kb, nullptr, d);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
}  // namespace vb

// Y[R, N] = X[R, K] * W[e(row block)]^T. b_mn = 0: W is [E, N, K]; b_mn = 1: W is [E, K, N] (the same storage read as the
// input-gradient operand: dX[R, N] = dY[R, K] * W[e] with W stored [E, K(out), N(in)]). Rows of unused blocks are not written.
extern "C" int vb_gemm_grouped(const void* A, const void* B, void* C, const int* blk_expert, int R, int N, int K, int E, int lda, int ldc,
                               int b_mn, int* err_word, cudaStream_t stream) {
  using namespace vb;
  if (R <= 0) return 0;
  if ((R % BM) != 0 || (lda & 7) || (N & 7) || (K & 7) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -4;
  return b_mn ? launch_grouped_fwd<true>(A, B, C, blk_expert, R, N, K, E, lda, ldc, err_word, stream)
              : launch_grouped_fwd<false>(A, B, C, blk_expert, R, N, K, E, lda, ldc, err_word, stream);
}

// Expert-parallel dispatch fused into the grouped GEMM: Y[R, N] = gather(X)[R, K] * W[e(row block)]^T where row r of the operand
// is fetched by the kernel's copy warps from src_ptrs[row_src[r] >> 24] (that rank's [*, K] token buffer, row stride ld_src,
// plain peer loads) into `stage` ([R, K] bf16, local) while the tensor cores work on blocks that have already arrived.
// stage_flags: R / 128 ints, zeroed here. After the call `stage` holds the gathered operand (the backward pass reuses it).
namespace vb {
template <bool B_MN>
static int launch_grouped_dispatch(const long* src_ptrs, int world, int ld_src, const int* row_src, const void* B, void* C, const int* blk_expert,
                                   int R, int N, int K, int E, int ldc, void* stage, int* stage_flags, int* err_word, cudaStream_t stream) {
  constexpr int BN = 256;
  using Cfg = GemmCfg<BN>;
  CUtensorMap tmA, tmB;
  if (make_tmap_2d(&tmA, stage, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, R, K, K, BM, BK)) return -1;
  int rc;
  if (!B_MN) rc = make_tmap_3d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, E, (uint64_t)K * 2, (uint64_t)N * K * 2, BK, BN, 1);
  else       rc = make_tmap_3d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, E, (uint64_t)N * 2, (uint64_t)N * K * 2, 64, BK, 1);
  if (rc) return rc;
  // the staged all-gather GEMMs share this instantiation and raise the attribute to Cfg::SMEM_BYTES only: set it on every call
  constexpr int SMEM = Cfg::SMEM_BYTES + DISPATCH_SMEM_BYTES;
  static_assert(SMEM <= 227 * 1024, "pipeline stages + dispatch ring exceed the shared memory of an SM");
  auto kern = gemm_bf16_kernel<BN, false, B_MN, EPI_STORE, 8>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) return -10;
  if (cudaMemsetAsync(stage_flags, 0, sizeof(int) * (R / BM), stream) != cudaSuccess) return -13;
  DistArgs d = {};
  d.group_mode = 1; d.num_experts = E; d.blk_expert = blk_expert;
  d.seg_mode = 4; d.row_src = row_src; d.ld_seg = ld_src; d.world = world;
  for (int r = 0; r < world; ++r) d.seg_ptr[r] = reinterpret_cast<const void*>(src_ptrs[r]);
  d.stage = stage; d.stage_flags = stage_flags; d.stage_epoch = 1; d.ld_stage = K;
  d.stage_map = tmA;
  const int units = (R / BM) * ((N + BN - 1) / BN);
  const int grid = units < num_sms() ? units : num_sms();
  const int num_kb = (K + BK - 1) / BK;
  kern<<<grid, 192 + 32 * 8, SMEM, stream>>>(tmA, tmB, C, nullptr, R, N, K, ldc, 0, err_word, LmHeadEpi{}, 1, num_kb, nullptr, d);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

template <bool B_MN>
static int launch_grouped_combine(const void* A, const void* B, const int* blk_expert, const int* row_dst, const float* row_w, const long* out_ptrs,
                                  int world, int R, int N, int K, int E, int lda, int ld_out, int* err_word, cudaStream_t stream) {
  constexpr int BN = 256;
  using Cfg = GemmCfg<BN>;
  CUtensorMap tmA, tmB;
  if (make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, R, K, lda, BM, BK)) return -1;
  int rc;
  if (!B_MN) rc = make_tmap_3d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, E, (uint64_t)K * 2, (uint64_t)N * K * 2, BK, BN, 1);
  else       rc = make_tmap_3d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, E, (uint64_t)N * 2, (uint64_t)N * K * 2, 64, BK, 1);
  if (rc) return rc;
  // (the plain peer-scatter GEMMs share this instantiation and set the attribute to Cfg::SMEM_BYTES only: set it on every call)
  constexpr int SMEM = Cfg::SMEM_BYTES + COMBINE_SMEM_BYTES;
  static_assert(SMEM <= 227 * 1024, "pipeline stages + combine lines exceed the shared memory of an SM");
  auto kern = gemm_bf16_kernel<BN, false, B_MN, EPI_PEER>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) return -10;
  DistArgs d = {};
  d.group_mode = 1; d.num_experts = E; d.blk_expert = blk_expert;
  d.world = world; d.row_dst = row_dst; d.row_w = row_w;
  for (int r = 0; r < world; ++r) d.peer_out[r] = reinterpret_cast<void*>(out_ptrs[r]);
  const int units = (R / BM) * ((N + BN - 1) / BN);
  const int grid = units < num_sms() ? units : num_sms();
  const int num_kb = (K + BK - 1) / BK;
  kern<<<grid, 192, SMEM, stream>>>(tmA, tmB, nullptr, nullptr, R, N, K, ld_out, 0, err_word, LmHeadEpi{}, 1, num_kb, nullptr, d);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
}  // namespace vb

extern "C" int vb_gemm_grouped_dispatch(const long* src_ptrs, int world, int ld_src, const int* row_src, const void* B, void* C,
                                        const int* blk_expert, int R, int N, int K, int E, int ldc, int b_mn, void* stage, int* stage_flags,
                                        int* err_word, cudaStream_t stream) {
  using namespace vb;
  if (R <= 0) return 0;
  if (world < 1 || world > MAX_TP || (R % BM) != 0 || (ld_src & 7) || (N & 7) || (K & 7) || (reinterpret_cast<uintptr_t>(B) & 15) ||
      (reinterpret_cast<uintptr_t>(stage) & 15) || stage == nullptr || stage_flags == nullptr)
    return -4;
  return b_mn ? launch_grouped_dispatch<true>(src_ptrs, world, ld_src, row_src, B, C, blk_expert, R, N, K, E, ldc, stage, stage_flags, err_word, stream)
              : launch_grouped_dispatch<false>(src_ptrs, world, ld_src, row_src, B, C, blk_expert, R, N, K, E, ldc, stage, stage_flags, err_word, stream);
}

// Combine fused into the grouped GEMM's epilogue: (A[R, K] * W[e(row block)]^T)[r] * row_w[r] is stored as row
// (row_dst[r] & 0xFFFFFF) of out_ptrs[row_dst[r] >> 24] (row stride ld_out, plain peer stores); rows with row_dst < 0 are dropped.
// The receivers sum their top-k slots afterwards (a barrier has to separate the two).
extern "C" int vb_gemm_grouped_combine(const void* A, const void* B, const int* blk_expert, const int* row_dst, const float* row_w,
                                       const long* out_ptrs, int world, int R, int N, int K, int E, int lda, int ld_out, int b_mn, int* err_word,
                                       cudaStream_t stream) {
  using namespace vb;
  if (R <= 0) return 0;
  if (world < 1 || world > MAX_TP || (R % BM) != 0 || (lda & 7) || (N % 64) != 0 || (K & 7) || (ld_out & 7) ||
      (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return -4;
  return b_mn ? launch_grouped_combine<true>(A, B, blk_expert, row_dst, row_w, out_ptrs, world, R, N, K, E, lda, ld_out, err_word, stream)
              : launch_grouped_combine<false>(A, B, blk_expert, row_dst, row_w, out_ptrs, world, R, N, K, E, lda, ld_out, err_word, stream);
}

// dW[e][M, N] (+)= dY[rows_e, M]^T * X[rows_e, N] for every expert; expert_rng[e] = (first 128-row block, end block).
extern "C" int vb_gemm_grouped_wgrad(const void* dY, const void* X, void* dW, const void* expert_rng, int R, int M, int N, int E, int ld_dy,
                                     int ld_x, int out_f32, int accumulate, int* err_word, cudaStream_t stream) {
  using namespace vb;
  if (R <= 0 || E <= 0) return 0;
  if ((R % BM) != 0 || (ld_dy & 7) || (ld_x & 7) || (M % BM) != 0) return -4;
  constexpr int BN = 256;
  using Cfg = GemmCfg<BN>;
  CUtensorMap tmA, tmB;
  if (make_tmap_2d(&tmA, dY, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, R, M, ld_dy, BK, 64)) return -1;
  if (make_tmap_2d(&tmB, X, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, R, N, ld_x, BK, 64)) return -1;
  static bool attr_set = false;
  auto kern = gemm_bf16_kernel<BN, true, true, EPI_STORE>;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess) return -10;
    attr_set = true;
  }
  DistArgs d = {};
  d.group_mode = 2; d.num_experts = E; d.expert_rng = reinterpret_cast<const int2*>(expert_rng);
  const long units = (long)E * (M / BM) * ((N + BN - 1) / BN);
  const int grid = units < num_sms() ? (int)units : num_sms();
  const int flags = (out_f32 ? GEMM_OUT_F32 : 0) | (accumulate ? GEMM_ACCUM : 0);
  kern<<<grid, 192, Cfg::SMEM_BYTES, stream>>>(tmA, tmB, dW, nullptr, M, N, R, N, flags, err_word, LmHeadEpi{}, 1, (R + BK - 1) / BK, nullptr, d);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Sequence → head all-to-all fused into the projection GEMM (Ulysses): this rank's [M, K] token shard times W[N, K]^T;
// output head h (head_dim columns) is written to rank head_rank[h]'s buffer at rows [row_off, row_off + M), head slot
// head_slot[h]. out_ptrs[r] = rank r's [T_total, ld_out] bf16 buffer.
extern "C" int vb_gemm_head_scatter(const void* A, const void* B, const void* bias, int M, int N, int K, int lda, int ldb, int ld_out,
                                    const long* out_ptrs, int world, int row_off, int head_dim, const int* head_rank, const int* head_slot,
                                    int b_mn, int* err_word, cudaStream_t st) {
  using namespace vb;
  if (world > MAX_TP || head_dim <= 0 || (head_dim % 32) != 0 || (N % head_dim) != 0 || N / head_dim > 192 || (ld_out & 7)) return -2;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda & 7) || (ldb & 7)) return -4;
  DistArgs d = {};
  d.world = world; d.row_off = row_off; d.head_dim = head_dim;
  for (int h = 0; h < N / head_dim; ++h) {
    if (head_rank[h] < 0 || head_rank[h] >= world || head_slot[h] < 0 || head_slot[h] > 0xFFF) return -2;
    d.head_map[h] = (uint16_t)((head_rank[h] << 12) | head_slot[h]);
  }
  for (int r = 0; r < world; ++r) d.peer_out[r] = reinterpret_cast<void*>(out_ptrs[r]);
  if (b_mn) return launch_dist<EPI_PEER, true>(pick_bn_dist(M, N), A, B, nullptr, bias, M, N, K, lda, ldb, ld_out, err_word, st, d);
  return launch_dist<EPI_PEER>(pick_bn_dist(M, N), A, B, nullptr, bias, M, N, K, lda, ldb, ld_out, err_word, st, d);
}

// Head → sequence all-to-all fused into the consuming GEMM (Ulysses output projection): C[M, N] = A B^T where the K axis
// of A is split over ranks: columns [r * k_per_rank, (r+1) * k_per_rank) are rows [row_off, row_off + M) of rank r's
// [T_total, k_per_rank] buffer (seg_ptrs[r], row stride ld_seg), read with TMA straight from that rank's memory.
extern "C" int vb_gemm_kseg(const long* seg_ptrs, int world, int k_per_rank, int ld_seg, int rows_total, int row_off, const void* B, int ldb,
                            void* C, const void* bias, int M, int N, int ldc, int rank, void* stage, int* stage_flags, int stage_epoch,
                            int b_mn, int* err_word, cudaStream_t st) {
  using namespace vb;
  if (world > MAX_TP || world < 1 || (k_per_rank % BK) != 0 || (ld_seg & 7) || (ldb & 7)) return -4;
  DistArgs d = {};
  d.seg_mode = 3; d.seg_rows = k_per_rank; d.n_seg = world; d.row_off = row_off;
  for (int r = 0; r < world; ++r) {
    if (make_tmap_2d(&d.seg[r], reinterpret_cast<const void*>(seg_ptrs[r]), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows_total, k_per_rank, ld_seg, BM, BK))
      return -1;
  }
  const int K = world * k_per_rank;
  if (stage != nullptr) {
    // `stage` is a local [ceil128(M), K] bf16 buffer (row stride K); `stage_flags` has ceil(M/128) * world ints
    if (rank < 0 || rank >= world) return -6;
    d.stage = stage; d.stage_flags = stage_flags; d.stage_epoch = stage_epoch; d.ld_stage = K; d.ld_seg = ld_seg; d.rank = rank;
    for (int r = 0; r < world; ++r) d.seg_ptr[r] = reinterpret_cast<const void*>(seg_ptrs[r]);
    if (make_tmap_2d(&d.stage_map, stage, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (M + 127) / 128 * 128, K, K, BM, BK)) return -1;
    if (cudaMemsetAsync(stage_flags, 0, sizeof(int) * ((M + 127) / 128) * world, st) != cudaSuccess) return -13;
  }
  if (b_mn)
    return launch_dist<EPI_STORE, true>(pick_bn_dist(M, N), reinterpret_cast<const void*>(seg_ptrs[0]), B, C, bias, M, N, K, ld_seg, ldb, ldc, err_word, st, d);
  return launch_dist<EPI_STORE>(pick_bn_dist(M, N), reinterpret_cast<const void*>(seg_ptrs[0]), B, C, bias, M, N, K, ld_seg, ldb, ldc, err_word, st, d);
}

// Signalled all-reduce in two launches: this GEMM writes its partial result (per K slice) into this rank's own symmetric
// buffer and its last CTA stores the new epoch into every peer's flag word; vb_slots_reduce_sig then waits for all ranks'
// flags, pulls their partials over NVLink and sums. sig_ptrs[r] = rank r's signal pad (>= 64 ints, zeroed once).
// K slice s of buffer half `parity` starts at parity * half_elems + s * slot_elems in this rank's OWN buffer (the slot sum
// pulls the peers' slices), so out_ptrs[r] must hold 2 * half_elems elements and split_k * slot_elems <= half_elems.
extern "C" void vb_allreduce_plan(int M, int N, int K, int* bn, int* split_k) {
  using namespace vb;
  // decode-sized M leaves few output tiles: slice K until (nearly) every SM streams its share of the weight
  const int num_m = (M + BM - 1) / BM;
  int best_bn = 128, best_s = 1;
  double best = 1e30;
  for (int b : {64, 128, 256}) {
    const int tiles = num_m * ((N + b - 1) / b);
    for (int s2 = 1; s2 <= 8; ++s2) {
      const int num_kb = (K + BK - 1) / BK;
      if (num_kb / s2 < 8) break;
      const int units = tiles * s2;
      const int waves = (units + num_sms() - 1) / num_sms();
      // per-unit cost: bytes staged through one SM (≈ 100 GB/s per SM) + fixed prologue/epilogue; slot traffic grows with s
      const double bytes = (double)(BM + b) * 2.0 * ((K + s2 - 1) / s2);
      const double t = waves * (bytes / 100e3 + 4.0) + 1.5 * s2;       // microseconds
      if (t < best) { best = t; best_bn = b; best_s = s2; }
    }
  }
  *bn = best_bn;
  *split_k = best_s;
}

extern "C" int vb_gemm_allreduce_sig(const void* A, const void* B, int M, int N, int K, int lda, int ldb, const long* out_ptrs,
                                     const long* sig_ptrs, int rank, int world, long slot_elems, long half_elems, int bn, int split_k,
                                     int* err_word, cudaStream_t st) {
  using namespace vb;
  if (world > MAX_TP || (N % 32) != 0) return -2;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda & 7) || (ldb & 7)) return -4;
  DistArgs d = {};
  d.rank = rank; d.world = world; d.rows_per_owner = 0; d.slot_elems = slot_elems;
  for (int r = 0; r < world; ++r) {
    d.peer_out[r] = reinterpret_cast<void*>(out_ptrs[r]);
    d.sig_peer[r] = reinterpret_cast<int*>(sig_ptrs[r]);
  }
  d.sig_local = reinterpret_cast<int*>(sig_ptrs[rank]);
  d.sig_half = half_elems;
  if ((long)split_k * slot_elems > half_elems) return -2;
  return launch_dist<EPI_PEER>(bn, A, B, nullptr, nullptr, M, N, K, lda, ldb, N, err_word, st, d, split_k);
}

extern "C" int vb_slots_reduce_sig(const long* slot_ptrs, const void* sig, int rank, int world, int split_k, long slot_elems, long half_elems,
                                   long rows, int cols, const void* residual, void* out, int ld_out, int* err_word, cudaStream_t st) {
  using namespace vb;
  if (cols % 8 || world > MAX_TP) return -2;
  long total = rows * (cols / 8);
  if (total == 0) return 0;
  PeerSlots ps = {};
  for (int r = 0; r < world; ++r) ps.p[r] = reinterpret_cast<const bf16*>(slot_ptrs[r]);
  int blocks = (int)((total + 255) / 256);
  if (blocks > num_sms() * 4) blocks = num_sms() * 4;
  slots_reduce_sig_kernel<<<blocks, 256, 0, st>>>(ps, (const int*)sig, rank, world, split_k, slot_elems, half_elems, rows, cols,
                                                  (const bf16*)residual, (bf16*)out, ld_out, err_word);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int vb_slots_reduce(const void* slots, int world, long slot_elems, long rows, int cols, int ld, const void* residual,
                               void* out, int ld_out, cudaStream_t st) {
  using namespace vb;
  if (cols % 8) return -2;
  long total = rows * (cols / 8);
  if (total == 0) return 0;
  int blocks = (int)((total + 255) / 256);
  if (blocks > num_sms() * 8) blocks = num_sms() * 8;
  slots_reduce_kernel<<<blocks, 256, 0, st>>>((const bf16*)slots, world, slot_elems, rows, cols, ld, (const bf16*)residual, (bf16*)out, ld_out);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
