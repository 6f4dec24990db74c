// RLHF loss-side kernels for sm_100a:
//   * token log-prob over the vocabulary (online log-sum-exp + gather) and its in-place backward
//   * PPO / GRPO clipped policy loss, DPO pair loss, masked value MSE  (forward value + d/dlogp)
//   * GAE reverse scan + masked whitening, GRPO group advantages
//   * Gumbel-max sampler fused with the sampled token's log-prob
//
// Math follows the reference's runtime: token log-probs are fp32 log_softmax + gather
// (RPEG/runtime/workers/megatron_worker.py:1879-1928), PPO targets and GAE are
// RPEG/runtime/ppo_math.py:14-92, the loss tuples are megatron_worker.py:4264-4274 (DPO),
// :4361-4387 (GRPO), :4388-4417 (PPO actor), :4650 (critic), group advantages :4418, and the
// sampler is megatron_worker.py:83-123.
#include "common.cuh"
#include "rpeg_kernels.h"

namespace rpeg {

constexpr int LP_THREADS = 256;

__device__ __forceinline__ void online_merge(float& m, float& s, float m2, float s2) {
  const float nm = fmaxf(m, m2);
  if (nm == -INFINITY) { m = nm; s = 0.f; return; }
  s = s * __expf(m - nm) + s2 * __expf(m2 - nm);
  m = nm;
}

__device__ __forceinline__ void block_lse(float& m, float& s, float* sm_m, float* sm_s) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
    online_merge(m, s, m2, s2);
  }
  if (lane == 0) { sm_m[warp] = m; sm_s[warp] = s; }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    m = lane < nw ? sm_m[lane] : -INFINITY;
    s = lane < nw ? sm_s[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
      online_merge(m, s, m2, s2);
    }
    if (lane == 0) { sm_m[0] = m; sm_s[0] = s; }
  }
  __syncthreads();
  m = sm_m[0];
  s = sm_s[0];
}

// One CTA per row. logp[t] = logits[t, y_t] - lse_t; lse saved for the backward.
// Rows with target < 0 get logp = 0 (ignored positions).
__global__ void __launch_bounds__(LP_THREADS)
token_logprob_fwd_kernel(const __nv_bfloat16* __restrict__ logits, const int* __restrict__ targets,
                         float* __restrict__ logp, float* __restrict__ lse_out, int V, int ld, float inv_temp) {
  __shared__ float sm_m[32], sm_s[32];
  const int row = blockIdx.x;
  const __nv_bfloat16* lr = logits + static_cast<size_t>(row) * ld;
  const uint4* lv = reinterpret_cast<const uint4*>(lr);
  const int nvec = V >> 3;
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < nvec; i += LP_THREADS) {
    const uint4 v = lv[i];
    const uint32_t* pv = reinterpret_cast<const uint32_t*>(&v);
    float x[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 a = unpack_bf16x2(pv[k]);
      x[2 * k] = a.x * inv_temp;
      x[2 * k + 1] = a.y * inv_temp;
    }
    float lm = x[0];
#pragma unroll
    for (int k = 1; k < 8; ++k) lm = fmaxf(lm, x[k]);
    float ls = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) ls += __expf(x[k] - lm);
    online_merge(m, s, lm, ls);
  }
  for (int i = (nvec << 3) + threadIdx.x; i < V; i += LP_THREADS) online_merge(m, s, __bfloat162float(lr[i]) * inv_temp, 1.f);
  block_lse(m, s, sm_m, sm_s);
  if (threadIdx.x == 0) {
    const float lse = m + __logf(s);
    lse_out[row] = lse;
    const int y = targets[row];
    logp[row] = (y >= 0 && y < V) ? __bfloat162float(lr[y]) * inv_temp - lse : 0.f;
  }
}

// In place: logits[t, v] <- coef[t] * (1[v == y_t] - exp(logits[t, v] - lse_t))   (bf16)
__global__ void __launch_bounds__(LP_THREADS)
token_logprob_bwd_kernel(__nv_bfloat16* __restrict__ logits, const int* __restrict__ targets,
                         const float* __restrict__ lse, const float* __restrict__ coef, int V, int ld,
                         float inv_temp) {
  const int row = blockIdx.x;
  __nv_bfloat16* lr = logits + static_cast<size_t>(row) * ld;
  uint4* lv = reinterpret_cast<uint4*>(lr);
  const int nvec = V >> 3;
  const float c = coef[row] * inv_temp, l = lse[row];
  const int y = targets[row];
  for (int i = threadIdx.x; i < nvec; i += LP_THREADS) {
    uint4 v = lv[i];
    uint32_t* pv = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 a = unpack_bf16x2(pv[k]);
      const int col = i * 8 + 2 * k;
      const float g0 = c * ((col == y ? 1.f : 0.f) - __expf(a.x * inv_temp - l));
      const float g1 = c * ((col + 1 == y ? 1.f : 0.f) - __expf(a.y * inv_temp - l));
      pv[k] = pack_bf16x2(g0, g1);
    }
    lv[i] = v;
  }
  for (int i = (nvec << 3) + threadIdx.x; i < V; i += LP_THREADS) {
    const float a = __bfloat162float(lr[i]);
    lr[i] = __float2bfloat16(c * ((i == y ? 1.f : 0.f) - __expf(a * inv_temp - l)));
  }
}

// Entropy of every row's softmax from the logits and the saved log-sum-exp: with x = logits / temperature and
// p_v = exp(x_v - lse), H = -sum_v p_v log p_v = lse - sum_v p_v x_v. One CTA per row (a second pass over the chunk's
// logits, taken only when the objective has an entropy bonus).
__global__ void __launch_bounds__(LP_THREADS)
token_entropy_kernel(const __nv_bfloat16* __restrict__ logits, const float* __restrict__ lse, float* __restrict__ ent,
                     int V, int ld, float inv_temp) {
  __shared__ float sm[32];
  const int row = blockIdx.x;
  const __nv_bfloat16* lr = logits + static_cast<size_t>(row) * ld;
  const uint4* lv = reinterpret_cast<const uint4*>(lr);
  const int nvec = V >> 3;
  const float l = lse[row];
  float acc = 0.f;
  for (int i = threadIdx.x; i < nvec; i += LP_THREADS) {
    const uint4 v = lv[i];
    const uint32_t* pv = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 a = unpack_bf16x2(pv[k]);
      const float x0 = a.x * inv_temp, x1 = a.y * inv_temp;
      acc += __expf(x0 - l) * x0 + __expf(x1 - l) * x1;
    }
  }
  for (int i = (nvec << 3) + threadIdx.x; i < V; i += LP_THREADS) {
    const float x = __bfloat162float(lr[i]) * inv_temp;
    acc += __expf(x - l) * x;
  }
  acc = warp_sum(acc);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) sm[warp] = acc;
  __syncthreads();
  if (warp == 0) {
    acc = lane < (LP_THREADS >> 5) ? sm[lane] : 0.f;
    acc = warp_sum(acc);
    if (lane == 0) ent[row] = l - acc;
  }
}

// In place, log-prob and entropy terms together:
//   logits[t, v] <- coef[t] * (1[v == y_t] - p_v) / temperature  -  ecoef[t] * p_v * (log p_v + H_t) / temperature
// (d H / d x_v = -p_v (log p_v + H); ecoef = d loss / d H per row, e.g. -entropy_coef * mask / denominator).
__global__ void __launch_bounds__(LP_THREADS)
token_logprob_entropy_bwd_kernel(__nv_bfloat16* __restrict__ logits, const int* __restrict__ targets,
                                 const float* __restrict__ lse, const float* __restrict__ coef,
                                 const float* __restrict__ ent, const float* __restrict__ ecoef, int V, int ld,
                                 float inv_temp) {
  const int row = blockIdx.x;
  __nv_bfloat16* lr = logits + static_cast<size_t>(row) * ld;
  uint4* lv = reinterpret_cast<uint4*>(lr);
  const int nvec = V >> 3;
  const float c = coef[row] * inv_temp, ec = ecoef[row] * inv_temp, l = lse[row], h = ent[row];
  const int y = targets[row];
  for (int i = threadIdx.x; i < nvec; i += LP_THREADS) {
    uint4 v = lv[i];
    uint32_t* pv = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 a = unpack_bf16x2(pv[k]);
      const int col = i * 8 + 2 * k;
      const float q0 = a.x * inv_temp - l, q1 = a.y * inv_temp - l;          // log p
      const float p0 = __expf(q0), p1 = __expf(q1);
      const float g0 = c * ((col == y ? 1.f : 0.f) - p0) - ec * p0 * (q0 + h);
      const float g1 = c * ((col + 1 == y ? 1.f : 0.f) - p1) - ec * p1 * (q1 + h);
      pv[k] = pack_bf16x2(g0, g1);
    }
    lv[i] = v;
  }
  for (int i = (nvec << 3) + threadIdx.x; i < V; i += LP_THREADS) {
    const float q = __bfloat162float(lr[i]) * inv_temp - l;
    const float p = __expf(q);
    lr[i] = __float2bfloat16(c * ((i == y ? 1.f : 0.f) - p) - ec * p * (q + h));
  }
}

// Clipped policy-gradient loss per token, PPO and GRPO in one kernel:
//   ratio = exp(lp - old);  pg = -min(ratio*A, clip(ratio, 1-eps, 1+eps)*A)
//   loss  = sum_t mask * (pg + kl_coef * (lp - ref)) * inv_denom
// acc[0] += loss, acc[1] += sum mask*(lp-ref), acc[2] += #clipped, acc[3] += sum mask*(old-lp) (approx KL)
// coef[t] = d loss / d lp[t].
__global__ void policy_loss_kernel(const float* __restrict__ lp, const float* __restrict__ old_lp,
                                   const float* __restrict__ ref_lp, const float* __restrict__ adv,
                                   const float* __restrict__ mask, float* __restrict__ coef,
                                   float* __restrict__ acc, long long n, float clip_eps, float kl_coef,
                                   float inv_denom) {
  float l_loss = 0.f, l_kl = 0.f, l_clip = 0.f, l_akl = 0.f;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float mk = mask[i];
    float c = 0.f;
    if (mk != 0.f) {
      const float x = lp[i], o = old_lp[i], a = adv[i];
      const float ratio = __expf(x - o);
      const float s1 = ratio * a;
      const float rc = fminf(fmaxf(ratio, 1.f - clip_eps), 1.f + clip_eps);
      const float s2 = rc * a;
      float g;
      if (s1 <= s2) { l_loss += -s1 * mk; g = -a * ratio; }
      else { l_loss += -s2 * mk; g = (rc == ratio) ? -a * ratio : 0.f; l_clip += mk; }
      if (ref_lp != nullptr && kl_coef != 0.f) {
        const float dkl = x - ref_lp[i];
        l_loss += kl_coef * dkl * mk;
        l_kl += dkl * mk;
        g += kl_coef;
      }
      l_akl += (o - x) * mk;
      c = g * mk * inv_denom;
    }
    coef[i] = c;
  }
  l_loss = warp_sum(l_loss); l_kl = warp_sum(l_kl); l_clip = warp_sum(l_clip); l_akl = warp_sum(l_akl);
  if ((threadIdx.x & 31) == 0) {
    atomicAdd(&acc[0], l_loss * inv_denom);
    atomicAdd(&acc[1], l_kl);
    atomicAdd(&acc[2], l_clip);
    atomicAdd(&acc[3], l_akl);
  }
}

// Masked row sums: out[b] = sum_t x[b, t] * mask[b, t]. One warp per row.
__global__ void masked_rowsum_kernel(const float* __restrict__ x, const float* __restrict__ mask,
                                     float* __restrict__ out, int B, int T) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= B) return;
  float s = 0.f;
  for (int t = threadIdx.x & 31; t < T; t += 32) s += x[static_cast<size_t>(row) * T + t] * mask[static_cast<size_t>(row) * T + t];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) out[row] = s;
}

// DPO over interleaved (chosen, rejected) rows: z = beta*((pi_c - pi_r) - (ref_c - ref_r));
// loss = mean_pairs -log sigmoid(z); seq_coef[2p] = -beta*sigmoid(-z)/P, seq_coef[2p+1] = +...
// acc[0] += loss, acc[1] += #(z>0) (preference accuracy), acc[2] += sum z/beta (reward margin).
__global__ void dpo_loss_kernel(const float* __restrict__ pi_seq, const float* __restrict__ ref_seq,
                                float* __restrict__ seq_coef, float* __restrict__ acc, int P, float beta) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  float l = 0.f, a = 0.f, mg = 0.f;
  if (p < P) {
    const float z = beta * ((pi_seq[2 * p] - pi_seq[2 * p + 1]) - (ref_seq[2 * p] - ref_seq[2 * p + 1]));
    // -log sigmoid(z) = softplus(-z), computed stably
    l = (z > 0.f ? 0.f : -z) + log1pf(__expf(-fabsf(z)));
    const float sneg = 1.f / (1.f + __expf(z));  // sigmoid(-z)
    seq_coef[2 * p] = -beta * sneg / static_cast<float>(P);
    seq_coef[2 * p + 1] = beta * sneg / static_cast<float>(P);
    a = z > 0.f ? 1.f : 0.f;
    mg = z / beta;
  }
  l = warp_sum(l); a = warp_sum(a); mg = warp_sum(mg);
  if ((threadIdx.x & 31) == 0) {
    atomicAdd(&acc[0], l / static_cast<float>(P));
    atomicAdd(&acc[1], a);
    atomicAdd(&acc[2], mg);
  }
}

// coef[b, t] = seq_coef[b] * mask[b, t]
__global__ void expand_seq_coef_kernel(const float* __restrict__ seq_coef, const float* __restrict__ mask,
                                       float* __restrict__ coef, long long n, int T) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) coef[i] = seq_coef[i / T] * mask[i];
}

// Masked value MSE: loss = sum mask*(v - ret)^2 * inv_denom; dv = 2*mask*(v - ret)*inv_denom.
__global__ void value_loss_kernel(const float* __restrict__ v, const float* __restrict__ ret,
                                  const float* __restrict__ mask, float* __restrict__ dv,
                                  float* __restrict__ acc, long long n, float inv_denom) {
  float l = 0.f;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float e = (v[i] - ret[i]) * mask[i];
    l += e * e;
    dv[i] = 2.f * e * inv_denom;
  }
  l = warp_sum(l);
  if ((threadIdx.x & 31) == 0) atomicAdd(&acc[0], l * inv_denom);
}

// GAE, one thread per row, reverse in time. Mask is binary, left aligned and contiguous.
//   r_t = -beta*(old_t - ref_t)*mask_t, + score at the last response token
//   delta_t = r_t + gamma*V_{t+1}*mask_{t+1} - V_t ; A_t = delta_t + gamma*lambda*mask_{t+1}*A_{t+1}
//   adv = A*mask ; ret = (A + V)*mask
__global__ void gae_kernel(const float* __restrict__ old_lp, const float* __restrict__ ref_lp,
                           const float* __restrict__ values, const float* __restrict__ mask,
                           const float* __restrict__ scores, float* __restrict__ adv, float* __restrict__ ret,
                           int B, int T, float beta, float gamma, float lambda) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const size_t o = static_cast<size_t>(b) * T;
  int last = -1;
  for (int t = T - 1; t >= 0; --t)
    if (mask[o + t] != 0.f) { last = t; break; }
  float a_next = 0.f, v_next = 0.f, m_next = 0.f;
  for (int t = T - 1; t >= 0; --t) {
    const float mk = mask[o + t];
    const float vt = values[o + t];
    float r = -beta * (old_lp[o + t] - (ref_lp ? ref_lp[o + t] : old_lp[o + t])) * mk;
    if (t == last) r += scores[b];
    const float delta = r + gamma * v_next * m_next - vt;
    const float a = delta + gamma * lambda * m_next * a_next;
    adv[o + t] = a * mk;
    ret[o + t] = (a + vt) * mk;
    a_next = a; v_next = vt; m_next = mk;
  }
}

// Masked whitening in place: x <- (x - mean) * rsqrt(var + 1e-6) * mask. Single CTA (n is B*T).
__global__ void masked_whiten_kernel(float* __restrict__ x, const float* __restrict__ mask, long long n) {
  __shared__ float red[3][32];
  float s = 0.f, c = 0.f;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) { s += x[i] * mask[i]; c += mask[i]; }
  s = warp_sum(s); c = warp_sum(c);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (lane == 0) { red[0][warp] = s; red[1][warp] = c; }
  __syncthreads();
  if (warp == 0) {
    s = lane < nw ? red[0][lane] : 0.f; c = lane < nw ? red[1][lane] : 0.f;
    s = warp_sum(s); c = warp_sum(c);
    if (lane == 0) { red[0][0] = s; red[1][0] = c; }
  }
  __syncthreads();
  const float cnt = fmaxf(red[1][0], 1.f);
  const float mean = red[0][0] / cnt;
  __syncthreads();
  float q = 0.f;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) { const float d = (x[i] - mean) * mask[i]; q += d * d; }
  q = warp_sum(q);
  if (lane == 0) red[2][warp] = q;
  __syncthreads();
  if (warp == 0) {
    q = lane < nw ? red[2][lane] : 0.f;
    q = warp_sum(q);
    if (lane == 0) red[2][0] = q;
  }
  __syncthreads();
  const float rs = rsqrtf(red[2][0] / cnt + 1e-6f);
  for (long long i = threadIdx.x; i < n; i += blockDim.x) x[i] = (x[i] - mean) * rs * mask[i];
}

// GRPO group advantages: rows are grouped K per prompt; a = (r - mean_g) / max(std_g, 1e-6) (biased).
__global__ void group_advantage_kernel(const float* __restrict__ rewards, float* __restrict__ out, int G, int K) {
  const int g = blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= G) return;
  float s = 0.f;
  for (int k = 0; k < K; ++k) s += rewards[g * K + k];
  const float mean = s / K;
  float q = 0.f;
  for (int k = 0; k < K; ++k) { const float d = rewards[g * K + k] - mean; q += d * d; }
  const float sd = fmaxf(sqrtf(q / K), 1e-6f);
  for (int k = 0; k < K; ++k) out[g * K + k] = (rewards[g * K + k] - mean) / sd;
}

// Stateless counter RNG -> uniform in (0,1).
__device__ __forceinline__ float hash_uniform(uint64_t seed, uint32_t row, uint32_t col) {
  uint64_t z = seed + 0x9E3779B97F4A7C15ull * (static_cast<uint64_t>(row) << 32 | col);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z = z ^ (z >> 31);
  return (static_cast<float>(z >> 40) + 0.5f) * (1.0f / 16777216.0f);
}

// One CTA per row: exact multinomial sample from softmax(logits/temp) by the Gumbel-max trick, in
// the same pass that builds the log-sum-exp, so the sampled token's log-prob costs nothing extra.
// greedy != 0 picks the argmax. `forced[row] >= 0` overrides the choice (used to inject EOS in
// synthetic workloads) while still reporting that token's log-prob.
__global__ void __launch_bounds__(LP_THREADS)
sample_kernel(const __nv_bfloat16* __restrict__ logits, int V, int ld, float inv_temp, int greedy,
              unsigned long long seed, const unsigned long long* __restrict__ seed_offset,
              const int* __restrict__ forced, int* __restrict__ token_out, float* __restrict__ logp_out) {
  griddep_launch();
  griddep_wait();   // may have been scheduled under the previous kernel's tail: nothing is read or written before this
  __shared__ float sm_m[32], sm_s[32], sm_best[32];
  __shared__ int sm_idx[32];
  const int row = blockIdx.x;
  // a device-resident offset (e.g. a step counter) keeps replays of a captured graph from reusing noise
  if (seed_offset != nullptr) seed += seed_offset[0] * 0xD1B54A32D192ED03ull;
  const __nv_bfloat16* lr = logits + static_cast<size_t>(row) * ld;
  float m = -INFINITY, s = 0.f, best = -INFINITY;
  int best_i = 0;
  auto take = [&](int i, float raw) {
    const float x = raw * inv_temp;
    online_merge(m, s, x, 1.f);
    float key = x;
    if (!greedy) key += -__logf(-__logf(hash_uniform(seed, row, i)));
    if (key > best || (key == best && i < best_i)) { best = key; best_i = i; }
  };
  if (((reinterpret_cast<uintptr_t>(lr) | static_cast<uintptr_t>(ld) * 2) & 15) == 0) {
    // 16-byte loads, two in flight per thread: the row is read at memory speed instead of one 2-byte load per
    // round trip (the noise of an element depends on its index only, so the result does not depend on the order)
    const uint4* lv = reinterpret_cast<const uint4*>(lr);
    const int nvec = V >> 3;
    for (int j = threadIdx.x; j < nvec; j += 2 * LP_THREADS) {
      const int j2 = j + LP_THREADS;
      const uint4 a = lv[j];
      uint4 b = make_uint4(0u, 0u, 0u, 0u);
      if (j2 < nvec) b = lv[j2];
      const uint32_t* pa = reinterpret_cast<const uint32_t*>(&a);
      const uint32_t* pb = reinterpret_cast<const uint32_t*>(&b);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = unpack_bf16x2(pa[e]);
        take(j * 8 + 2 * e, f.x);
        take(j * 8 + 2 * e + 1, f.y);
      }
      if (j2 < nvec) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = unpack_bf16x2(pb[e]);
          take(j2 * 8 + 2 * e, f.x);
          take(j2 * 8 + 2 * e + 1, f.y);
        }
      }
    }
    for (int i = (nvec << 3) + threadIdx.x; i < V; i += LP_THREADS) take(i, __bfloat162float(lr[i]));
  } else {
    for (int i = threadIdx.x; i < V; i += LP_THREADS) take(i, __bfloat162float(lr[i]));
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float b2 = __shfl_xor_sync(0xffffffffu, best, o);
    const int i2 = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (b2 > best || (b2 == best && i2 < best_i)) { best = b2; best_i = i2; }
  }
  if (lane == 0) { sm_best[warp] = best; sm_idx[warp] = best_i; }
  block_lse(m, s, sm_m, sm_s);  // contains __syncthreads
  if (threadIdx.x == 0) {
    const int nw = blockDim.x >> 5;
    for (int w = 1; w < nw; ++w)
      if (sm_best[w] > best || (sm_best[w] == best && sm_idx[w] < best_i)) { best = sm_best[w]; best_i = sm_idx[w]; }
    if (forced != nullptr && forced[row] >= 0) best_i = forced[row];
    token_out[row] = best_i;
    logp_out[row] = __bfloat162float(lr[best_i]) * inv_temp - (m + __logf(s));
  }
}

// Sampling restricted to the top-k tokens and/or the smallest set whose probability mass reaches top_p.
// Both cut-offs are found as a threshold on the (temperature-scaled) logit by bisection: for a candidate
// threshold one pass over the row counts the tokens above it and adds up their probability, so no sort
// and no scratch memory is needed (26 passes over a row that stays in L1/L2). The token is then drawn by
// Gumbel-max among the survivors. The reported log-prob is taken under the FULL softmax, which is what the
// training passes recompute. top_k <= 0 and top_p >= 1 switch the respective filter off.
__global__ void __launch_bounds__(LP_THREADS)
sample_filtered_kernel(const __nv_bfloat16* __restrict__ logits, int V, int ld, float inv_temp, int top_k, float top_p,
                       unsigned long long seed, const unsigned long long* __restrict__ seed_offset,
                       const int* __restrict__ forced, int* __restrict__ token_out, float* __restrict__ logp_out) {
  __shared__ float sm_m[32], sm_s[32], sm_best[32], sm_cnt[32], sm_mass[32];
  __shared__ int sm_idx[32];
  __shared__ float sm_bc[2];
  const int row = blockIdx.x;
  if (seed_offset != nullptr) seed += seed_offset[0] * 0xD1B54A32D192ED03ull;
  const __nv_bfloat16* lr = logits + static_cast<size_t>(row) * ld;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < V; i += LP_THREADS) online_merge(m, s, __bfloat162float(lr[i]) * inv_temp, 1.f);
  block_lse(m, s, sm_m, sm_s);                       // m, s now hold the row's max and sum(exp(x - m)) in every thread
  const float lse = m + __logf(s);
  const bool use_k = top_k > 0 && top_k < V, use_p = top_p < 1.f;
  float lo_k = m - 40.f, hi_k = m, lo_p = m - 40.f, hi_p = m;
  if (use_k || use_p) {
    for (int it = 0; it < 26; ++it) {
      const float mid_k = 0.5f * (lo_k + hi_k), mid_p = 0.5f * (lo_p + hi_p);
      float cnt = 0.f, mass = 0.f;
      for (int i = threadIdx.x; i < V; i += LP_THREADS) {
        const float x = __bfloat162float(lr[i]) * inv_temp;
        cnt += x >= mid_k ? 1.f : 0.f;
        mass += x >= mid_p ? __expf(x - lse) : 0.f;
      }
      cnt = warp_sum(cnt);
      mass = warp_sum(mass);
      __syncthreads();
      if (lane == 0) { sm_cnt[warp] = cnt; sm_mass[warp] = mass; }
      __syncthreads();
      if (threadIdx.x == 0) {
        float c = 0.f, p = 0.f;
        for (int w = 0; w < nw; ++w) { c += sm_cnt[w]; p += sm_mass[w]; }
        sm_bc[0] = c; sm_bc[1] = p;
      }
      __syncthreads();
      if (sm_bc[0] >= static_cast<float>(top_k)) lo_k = mid_k; else hi_k = mid_k;     // still at least k tokens above: raise the bar
      if (sm_bc[1] >= top_p) lo_p = mid_p; else hi_p = mid_p;                          // still at least top_p mass above
    }
  }
  float thr = -INFINITY;
  if (use_k) thr = fmaxf(thr, lo_k);
  if (use_p) thr = fmaxf(thr, lo_p);
  float best = -INFINITY;
  int best_i = 0;
  for (int i = threadIdx.x; i < V; i += LP_THREADS) {
    const float x = __bfloat162float(lr[i]) * inv_temp;
    if (x < thr) continue;
    const float key = x - __logf(-__logf(hash_uniform(seed, row, i)));
    if (key > best) { best = key; best_i = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float b2 = __shfl_xor_sync(0xffffffffu, best, o);
    const int i2 = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (b2 > best || (b2 == best && i2 < best_i)) { best = b2; best_i = i2; }
  }
  __syncthreads();
  if (lane == 0) { sm_best[warp] = best; sm_idx[warp] = best_i; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < nw; ++w)
      if (sm_best[w] > best || (sm_best[w] == best && sm_idx[w] < best_i)) { best = sm_best[w]; best_i = sm_idx[w]; }
    if (forced != nullptr && forced[row] >= 0) best_i = forced[row];
    token_out[row] = best_i;
    logp_out[row] = __bfloat162float(lr[best_i]) * inv_temp - lse;
  }
}

// Value / reward head: out[t] = dot(h[t, :], w) + bias. One warp per row.
__global__ void head_gemv_kernel(const __nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ w,
                                 const float* __restrict__ bias, float* __restrict__ out, int T, int d) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= T) return;
  const uint4* hr = reinterpret_cast<const uint4*>(h + static_cast<size_t>(row) * d);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  float s = 0.f;
  for (int i = threadIdx.x & 31; i < (d >> 3); i += 32) {
    const uint4 a = hr[i], b = wr[i];
    const uint32_t *pa = reinterpret_cast<const uint32_t*>(&a), *pb = reinterpret_cast<const uint32_t*>(&b);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 x = unpack_bf16x2(pa[k]), y = unpack_bf16x2(pb[k]);
      s += x.x * y.x + x.y * y.y;
    }
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) out[row] = s + (bias ? bias[0] : 0.f);
}

// Backward of the scalar head: dh[t, :] = dout[t] * w ; dw += sum_t dout[t] * h[t, :] ; db += sum dout.
__global__ void head_gemv_bwd_kernel(const __nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ w,
                                     const float* __restrict__ dout, __nv_bfloat16* __restrict__ dh,
                                     float* __restrict__ dw, float* __restrict__ db, int T, int d,
                                     int rows_per_cta) {
  // thread owns columns {threadIdx.x*2, +1} + k*2*blockDim
  const int row0 = blockIdx.x * rows_per_cta, row1 = min(T, row0 + rows_per_cta);
  float lb = 0.f;
  for (int c = threadIdx.x * 2; c < d; c += blockDim.x * 2) {
    const float2 wv = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(w + c));
    float a0 = 0.f, a1 = 0.f;
    for (int r = row0; r < row1; ++r) {
      const float g = dout[r];
      const float2 hv = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(h + static_cast<size_t>(r) * d + c));
      a0 += g * hv.x; a1 += g * hv.y;
      *reinterpret_cast<uint32_t*>(dh + static_cast<size_t>(r) * d + c) = pack_bf16x2(g * wv.x, g * wv.y);
    }
    atomicAdd(&dw[c], a0);
    atomicAdd(&dw[c + 1], a1);
  }
  if (threadIdx.x == 0 && db != nullptr) {
    for (int r = row0; r < row1; ++r) lb += dout[r];
    atomicAdd(db, lb);
  }
}

}  // namespace rpeg

using namespace rpeg;
#define STREAM(s) reinterpret_cast<cudaStream_t>(s)
#define LAUNCH_OK() (cudaGetLastError() == cudaSuccess ? 0 : -21)
static inline unsigned grid_for(long long n, int block, int cap = 148 * 16) {
  long long g = (n + block - 1) / block;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return static_cast<unsigned>(g);
}

extern "C" int rpeg_token_logprob_fwd(const void* logits, const int* targets, float* logp, float* lse, int T,
                                      int V, int ld, float temperature, void* stream) {
  if (T <= 0) return 0;
  if (ld & 7) return -2;
  token_logprob_fwd_kernel<<<T, LP_THREADS, 0, STREAM(stream)>>>(static_cast<const __nv_bfloat16*>(logits), targets,
                                                                logp, lse, V, ld, 1.f / temperature);
  return LAUNCH_OK();
}
extern "C" int rpeg_token_logprob_bwd(void* logits, const int* targets, const float* lse, const float* coef,
                                      int T, int V, int ld, float temperature, void* stream) {
  if (T <= 0) return 0;
  if (ld & 7) return -2;
  token_logprob_bwd_kernel<<<T, LP_THREADS, 0, STREAM(stream)>>>(static_cast<__nv_bfloat16*>(logits), targets, lse,
                                                                coef, V, ld, 1.f / temperature);
  return LAUNCH_OK();
}
extern "C" int rpeg_token_entropy(const void* logits, const float* lse, float* ent, int T, int V, int ld,
                                  float temperature, void* stream) {
  if (T <= 0) return 0;
  if (ld & 7) return -2;
  token_entropy_kernel<<<T, LP_THREADS, 0, STREAM(stream)>>>(static_cast<const __nv_bfloat16*>(logits), lse, ent, V, ld,
                                                            1.f / temperature);
  return LAUNCH_OK();
}
extern "C" int rpeg_token_logprob_entropy_bwd(void* logits, const int* targets, const float* lse, const float* coef,
                                              const float* ent, const float* ecoef, int T, int V, int ld,
                                              float temperature, void* stream) {
  if (T <= 0) return 0;
  if (ld & 7) return -2;
  token_logprob_entropy_bwd_kernel<<<T, LP_THREADS, 0, STREAM(stream)>>>(static_cast<__nv_bfloat16*>(logits), targets, lse,
                                                                        coef, ent, ecoef, V, ld, 1.f / temperature);
  return LAUNCH_OK();
}
extern "C" int rpeg_policy_loss(const float* lp, const float* old_lp, const float* ref_lp, const float* adv,
                                const float* mask, float* coef, float* acc, long long n, float clip_eps,
                                float kl_coef, float inv_denom, void* stream) {
  if (n <= 0) return 0;
  policy_loss_kernel<<<grid_for(n, 256), 256, 0, STREAM(stream)>>>(lp, old_lp, ref_lp, adv, mask, coef, acc, n,
                                                                  clip_eps, kl_coef, inv_denom);
  return LAUNCH_OK();
}
extern "C" int rpeg_masked_rowsum(const float* x, const float* mask, float* out, int B, int T, void* stream) {
  if (B <= 0) return 0;
  masked_rowsum_kernel<<<(B + 3) / 4, 128, 0, STREAM(stream)>>>(x, mask, out, B, T);
  return LAUNCH_OK();
}
extern "C" int rpeg_dpo_loss(const float* pi_seq, const float* ref_seq, float* seq_coef, float* acc, int P,
                             float beta, void* stream) {
  if (P <= 0) return 0;
  dpo_loss_kernel<<<(P + 127) / 128, 128, 0, STREAM(stream)>>>(pi_seq, ref_seq, seq_coef, acc, P, beta);
  return LAUNCH_OK();
}
extern "C" int rpeg_expand_seq_coef(const float* seq_coef, const float* mask, float* coef, int B, int T,
                                    void* stream) {
  const long long n = static_cast<long long>(B) * T;
  if (n <= 0) return 0;
  expand_seq_coef_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, STREAM(stream)>>>(seq_coef, mask, coef, n, T);
  return LAUNCH_OK();
}
extern "C" int rpeg_value_loss(const float* v, const float* ret, const float* mask, float* dv, float* acc,
                               long long n, float inv_denom, void* stream) {
  if (n <= 0) return 0;
  value_loss_kernel<<<grid_for(n, 256), 256, 0, STREAM(stream)>>>(v, ret, mask, dv, acc, n, inv_denom);
  return LAUNCH_OK();
}
extern "C" int rpeg_gae(const float* old_lp, const float* ref_lp, const float* values, const float* mask,
                        const float* scores, float* adv, float* ret, int B, int T, float beta, float gamma,
                        float lambda, int whiten, void* stream) {
  if (B <= 0) return 0;
  gae_kernel<<<(B + 63) / 64, 64, 0, STREAM(stream)>>>(old_lp, ref_lp, values, mask, scores, adv, ret, B, T, beta,
                                                      gamma, lambda);
  if (whiten) masked_whiten_kernel<<<1, 1024, 0, STREAM(stream)>>>(adv, mask, static_cast<long long>(B) * T);
  return LAUNCH_OK();
}
extern "C" int rpeg_group_advantage(const float* rewards, float* out, int G, int K, void* stream) {
  if (G <= 0) return 0;
  group_advantage_kernel<<<(G + 63) / 64, 64, 0, STREAM(stream)>>>(rewards, out, G, K);
  return LAUNCH_OK();
}
extern "C" int rpeg_sample(const void* logits, int B, int V, int ld, float temperature, int greedy,
                           unsigned long long seed, const unsigned long long* seed_offset, const int* forced,
                           int* token_out, float* logp_out, void* stream) {
  if (B <= 0) return 0;
  launch_pdl(sample_kernel, dim3(B), dim3(LP_THREADS), 0, STREAM(stream), static_cast<const __nv_bfloat16*>(logits), V, ld,
                                                     1.f / temperature, greedy, seed, seed_offset, forced, token_out, logp_out);
  return LAUNCH_OK();
}
extern "C" int rpeg_sample_filtered(const void* logits, int B, int V, int ld, float temperature, int top_k, float top_p,
                                    unsigned long long seed, const unsigned long long* seed_offset, const int* forced,
                                    int* token_out, float* logp_out, void* stream) {
  if (B <= 0) return 0;
  if (!(temperature > 0.f) || !(top_p > 0.f)) return -2;
  sample_filtered_kernel<<<B, LP_THREADS, 0, STREAM(stream)>>>(static_cast<const __nv_bfloat16*>(logits), V, ld, 1.f / temperature,
                                                              top_k, top_p, seed, seed_offset, forced, token_out, logp_out);
  return LAUNCH_OK();
}
extern "C" int rpeg_head_gemv(const void* h, const void* w, const float* bias, float* out, int T, int d,
                              void* stream) {
  if (T <= 0) return 0;
  if (d & 7) return -2;
  head_gemv_kernel<<<(T + 3) / 4, 128, 0, STREAM(stream)>>>(static_cast<const __nv_bfloat16*>(h),
                                                           static_cast<const __nv_bfloat16*>(w), bias, out, T, d);
  return LAUNCH_OK();
}
extern "C" int rpeg_head_gemv_bwd(const void* h, const void* w, const float* dout, void* dh, float* dw,
                                  float* db, int T, int d, void* stream) {
  if (T <= 0) return 0;
  if (d & 1) return -2;
  const int rows_per_cta = 64;
  head_gemv_bwd_kernel<<<(T + rows_per_cta - 1) / rows_per_cta, 256, 0, STREAM(stream)>>>(
      static_cast<const __nv_bfloat16*>(h), static_cast<const __nv_bfloat16*>(w), dout,
      static_cast<__nv_bfloat16*>(dh), dw, db, T, d, rows_per_cta);
  return LAUNCH_OK();
}
