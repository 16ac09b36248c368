// RL-specific elementwise kernels: the PPO/GRPO clipped policy loss with its KL-to-reference term (forward value,
// gradient with respect to the log-probs and the logging statistics in ONE pass over the response window), and the
// GRPO group-normalised advantage. The PyTorch formulations they replace launch ~40 small kernels per micro-batch
// (verl/trainer/ppo/core_algos.py:1165-1250 compute_policy_loss_vanilla, :2205-2260 kl_penalty, :1100-1160 agg_loss,
// :267-331 compute_grpo_outcome_advantage).
#include "common.cuh"

namespace vb {

// kl_type: 0 none, 1 "kl" (k1 = lp - ref), 2 "abs", 3 "mse" (k2 = 0.5 d^2), 4 "low_var_kl" (k3, clamped to +-10)
// Per token i with weight w_i (aggregation weight, 0 on masked tokens):
//   loss += w_i * (pg_i * is_i + kl_coef * kl_i);  grad_i = w_i * d(...)/d lp_i
// stats[0] += w-independent masked sums: [0] clipped-high count, [1] sum(-(lp-old)), [2] clipped-lower count,
//   [3] sum kl, [4] masked token count, [5] sum pg (weighted), [6] sum kl (weighted)
__global__ void __launch_bounds__(256) ppo_loss_kernel(const float* __restrict__ lp, const float* __restrict__ old_lp,
                                                       const float* __restrict__ ref_lp, const float* __restrict__ adv,
                                                       const float* __restrict__ weight, const float* __restrict__ mask,
                                                       const float* __restrict__ is_w, long n, float clip_lo, float clip_hi, float clip_c,
                                                       int kl_type, float kl_coef, float* __restrict__ grad,
                                                       float* __restrict__ loss_out, float* __restrict__ stats) {
  float acc[7] = {0, 0, 0, 0, 0, 0, 0};
  float loss = 0.f;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const float m = mask[i];
    const float w = weight[i];
    const float x = lp[i];
    const float a = adv[i];
    const float d = fminf(fmaxf(x - old_lp[i], -20.f), 20.f);
    const bool d_live = (x - old_lp[i]) > -20.f && (x - old_lp[i]) < 20.f;     // clamp passes gradient only inside
    const float ratio = __expf(d);
    const float l1 = -a * ratio;
    const float rc = fminf(fmaxf(ratio, 1.f - clip_lo), 1.f + clip_hi);
    const float l2 = -a * rc;
    const bool use2 = l2 > l1;                       // max(l1, l2): the clipped branch has zero gradient
    float pg = use2 ? l2 : l1;
    float dpg = (use2 || !d_live) ? 0.f : -a * ratio;
    bool lower = false;
    if (a < 0.f) {
      const float l3 = -a * clip_c;
      if (pg > l3) {                                 // dual clip: min(l3, pg), constant branch
        lower = true;
        pg = l3;
        dpg = 0.f;
      }
    }
    const float isw = is_w != nullptr ? is_w[i] : 1.f;
    pg *= isw;
    dpg *= isw;
    float kl = 0.f, dkl = 0.f;
    if (kl_type != 0) {
      const float r = ref_lp[i];
      if (kl_type == 1) { kl = x - r; dkl = 1.f; }
      else if (kl_type == 2) { kl = fabsf(x - r); dkl = (x > r) ? 1.f : ((x < r) ? -1.f : 0.f); }
      else if (kl_type == 3) { kl = 0.5f * (x - r) * (x - r); dkl = x - r; }
      else {
        const float t = fminf(fmaxf(r - x, -20.f), 20.f);
        const bool t_live = (r - x) > -20.f && (r - x) < 20.f;
        const float e = __expf(t);
        const float k3 = e - t - 1.f;
        kl = fminf(fmaxf(k3, -10.f), 10.f);
        dkl = (k3 > -10.f && k3 < 10.f && t_live) ? (1.f - e) : 0.f;
      }
    }
    loss += w * (pg + kl_coef * kl);
    grad[i] = w * (dpg + kl_coef * dkl);
    acc[0] += m * (use2 ? 1.f : 0.f);
    acc[1] += m * (-d);
    acc[2] += m * (lower ? 1.f : 0.f);
    acc[3] += m * kl;
    acc[4] += m;
    acc[5] += w * pg;
    acc[6] += w * kl;
  }
  __shared__ float red[8][8];
  loss = warp_sum(loss);
#pragma unroll
  for (int k = 0; k < 7; ++k) acc[k] = warp_sum(acc[k]);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    red[warp][7] = loss;
    for (int k = 0; k < 7; ++k) red[warp][k] = acc[k];
  }
  __syncthreads();
  if (threadIdx.x < 8) {
    float s = 0.f;
    for (int wv = 0; wv < 8; ++wv) s += red[wv][threadIdx.x];
    if (threadIdx.x == 7) atomicAdd(loss_out, s);
    else atomicAdd(stats + threadIdx.x, s);
  }
}

// GRPO outcome advantage. scores [B] (sum of token rewards per trajectory), group [B] dense group ids in [0, G).
// Pass 1 (one block): per-group count / mean / unbiased std; pass 2: adv[b, t] = (score_b - mean_g) / (std_g + eps) * mask.
__global__ void grpo_group_stats_kernel(const float* __restrict__ scores, const int* __restrict__ group, int B, int G,
                                        float* __restrict__ mean, float* __restrict__ stdv) {
  extern __shared__ float sh[];        // [G] sum, [G] sumsq, [G] count
  float* s1 = sh;
  float* s2 = sh + G;
  float* cn = sh + 2 * G;
  for (int g = threadIdx.x; g < 3 * G; g += blockDim.x) sh[g] = 0.f;
  __syncthreads();
  for (int b = threadIdx.x; b < B; b += blockDim.x) {
    const int g = group[b];
    atomicAdd(&s1[g], scores[b]);
    atomicAdd(&cn[g], 1.f);
  }
  __syncthreads();
  for (int g = threadIdx.x; g < G; g += blockDim.x) s1[g] = cn[g] > 0.f ? s1[g] / cn[g] : 0.f;   // mean
  __syncthreads();
  for (int b = threadIdx.x; b < B; b += blockDim.x) {
    const int g = group[b];
    const float d = scores[b] - s1[g];
    atomicAdd(&s2[g], d * d);
  }
  __syncthreads();
  for (int g = threadIdx.x; g < G; g += blockDim.x) {
    if (cn[g] <= 1.f) {                 // a group of one keeps its raw score: mean 0, std 1
      mean[g] = 0.f;
      stdv[g] = 1.f;
    } else {
      mean[g] = s1[g];
      stdv[g] = sqrtf(s2[g] / (cn[g] - 1.f));
    }
  }
}

__global__ void grpo_advantage_kernel(const float* __restrict__ scores, const int* __restrict__ group, const float* __restrict__ mean,
                                      const float* __restrict__ stdv, const float* __restrict__ mask, int B, int R, float eps,
                                      int norm_by_std, float* __restrict__ adv) {
  const long n = (long)B * R;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const int b = i / R;
    const int g = group[b];
    float a = scores[b] - mean[g];
    if (norm_by_std) a /= (stdv[g] + eps);
    adv[i] = a * mask[i];
  }
}


// ---------------------------------------------------------------- GAE (generalised advantage estimation)
// One thread per trajectory walks its response window backwards; masked positions carry the running state through
// (reference semantics: verl/trainer/ppo/core_algos.py compute_gae_advantage_return). Also accumulates the masked sum and sum of
// squares of the advantages (stats[0..2] = sum, sum of squares, count) for the whitening pass.
__global__ void gae_kernel(const float* __restrict__ rewards, const float* __restrict__ values, const float* __restrict__ mask, int B, int R,
                           float gamma, float lam, float* __restrict__ adv, float* __restrict__ ret, float* __restrict__ stats) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  float s = 0.f, s2 = 0.f, n = 0.f;
  if (b < B) {
    const long o = (long)b * R;
    float nextv = 0.f, last = 0.f;
    for (int t = R - 1; t >= 0; --t) {
      const float v = values[o + t], m = mask[o + t];
      const float delta = rewards[o + t] + gamma * nextv - v;
      const float cand = delta + gamma * lam * last;
      nextv = v * m + (1.f - m) * nextv;
      last = cand * m + (1.f - m) * last;
      adv[o + t] = last;
      ret[o + t] = last + v;
      s += last * m;
      s2 += last * last * m;
      n += m;
    }
  }
  s = warp_sum(s); s2 = warp_sum(s2); n = warp_sum(n);
  if ((threadIdx.x & 31) == 0) {
    atomicAdd(stats, s);
    atomicAdd(stats + 1, s2);
    atomicAdd(stats + 2, n);
  }
}

// (x - mean) * rsqrt(var_unbiased + 1e-8) with the masked moments of stats (two-pass variance from the raw moments in fp32
// would cancel badly for large means, so the second moment is recentred here: var = E[x^2] - mean^2 is only used when the
// caller passes centred data; for GAE advantages the mean is small against the spread).
__global__ void whiten_kernel(float* __restrict__ x, long n, const float* __restrict__ stats) {
  const float cnt = stats[2];
  const float mean = stats[0] / fmaxf(cnt, 1.f);
  float var = stats[1] / fmaxf(cnt, 1.f) - mean * mean;
  var = fmaxf(var, 0.f) * (cnt > 1.f ? cnt / (cnt - 1.f) : 1.f);
  const float r = rsqrtf(var + 1e-8f);
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) x[i] = (x[i] - mean) * r;
}

// ---------------------------------------------------------------- clipped value loss (forward value, gradient and clip fraction in one pass)
// per token: l = 0.5 * max((v - R)^2, (clip(v, v_old - c, v_old + c) - R)^2) * weight; grad = dl/dv; stats[0] = weighted sum,
// stats[1] = number of masked tokens where the clipped branch is the larger one, stats[2] = masked tokens.
__global__ void __launch_bounds__(256) value_loss_kernel(const float* __restrict__ v, const float* __restrict__ v_old, const float* __restrict__ ret,
                                                         const float* __restrict__ weight, const float* __restrict__ mask, long n, float clip,
                                                         float* __restrict__ grad, float* __restrict__ stats) {
  float loss = 0.f, nclip = 0.f, ntok = 0.f;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const float x = v[i], o = v_old[i], r = ret[i], w = weight[i], m = mask[i];
    const float c = fminf(fmaxf(x, o - clip), o + clip);
    const float l1 = (x - r) * (x - r), l2 = (c - r) * (c - r);
    const bool use2 = l2 > l1;
    loss += 0.5f * (use2 ? l2 : l1) * w;
    // the clipped branch has a gradient only where the clip is inactive (c == x)
    const float g = use2 ? ((c == x) ? (c - r) : 0.f) : (x - r);
    grad[i] = g * w;
    nclip += use2 ? m : 0.f;
    ntok += m;
  }
  loss = warp_sum(loss); nclip = warp_sum(nclip); ntok = warp_sum(ntok);
  if ((threadIdx.x & 31) == 0) {
    atomicAdd(stats, loss);
    atomicAdd(stats + 1, nclip);
    atomicAdd(stats + 2, ntok);
  }
}

}  // namespace vb

using namespace vb;

extern "C" {

// loss_out[1] and stats[7] must be zeroed by the caller.
int vb_ppo_loss(const float* lp, const float* old_lp, const float* ref_lp, const float* adv, const float* weight, const float* mask,
                const float* is_w, long n, float clip_lo, float clip_hi, float clip_c, int kl_type, float kl_coef, float* grad,
                float* loss_out, float* stats, cudaStream_t st) {
  if (n <= 0) return 0;
  if (kl_type != 0 && ref_lp == nullptr) return -2;
  long blocks = (n + 255) / 256;
  if (blocks > 148 * 4) blocks = 148 * 4;
  ppo_loss_kernel<<<(int)blocks, 256, 0, st>>>(lp, old_lp, ref_lp, adv, weight, mask, is_w, n, clip_lo, clip_hi, clip_c, kl_type, kl_coef, grad,
                                               loss_out, stats);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int vb_grpo_advantage(const float* scores, const int* group, int B, int G, const float* mask, int R, float eps, int norm_by_std,
                      float* mean, float* stdv, float* adv, cudaStream_t st) {
  if (B <= 0) return 0;
  if (G <= 0 || 3 * G * sizeof(float) > 200 * 1024) return -2;
  const size_t sh = 3 * (size_t)G * sizeof(float);
  if (sh > 48 * 1024) cudaFuncSetAttribute(grpo_group_stats_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sh);
  grpo_group_stats_kernel<<<1, 1024, sh, st>>>(scores, group, B, G, mean, stdv);
  long n = (long)B * R;
  long blocks = (n + 255) / 256;
  if (blocks > 148 * 4) blocks = 148 * 4;
  grpo_advantage_kernel<<<(int)blocks, 256, 0, st>>>(scores, group, mean, stdv, mask, B, R, eps, norm_by_std, adv);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// adv / ret [B, R]; stats[3] zeroed by the caller; whiten != 0 normalises adv in place with its masked moments.
int vb_gae(const float* rewards, const float* values, const float* mask, int B, int R, float gamma, float lam, int whiten, float* adv, float* ret,
           float* stats, cudaStream_t st) {
  if (B <= 0 || R <= 0) return 0;
  gae_kernel<<<(B + 127) / 128, 128, 0, st>>>(rewards, values, mask, B, R, gamma, lam, adv, ret, stats);
  if (whiten) {
    long n = (long)B * R;
    long blocks = (n + 255) / 256;
    if (blocks > 148 * 4) blocks = 148 * 4;
    whiten_kernel<<<(int)blocks, 256, 0, st>>>(adv, n, stats);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// stats[3] zeroed by the caller.
int vb_value_loss(const float* v, const float* v_old, const float* ret, const float* weight, const float* mask, long n, float clip, float* grad,
                  float* stats, cudaStream_t st) {
  if (n <= 0) return 0;
  long blocks = (n + 255) / 256;
  if (blocks > 148 * 4) blocks = 148 * 4;
  value_loss_kernel<<<(int)blocks, 256, 0, st>>>(v, v_old, ret, weight, mask, n, clip, grad, stats);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // extern "C"
