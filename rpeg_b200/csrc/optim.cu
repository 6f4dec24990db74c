// Optimizer-side kernels for sm_100a.
//
// Single GPU: fused AdamW on fp32 master weights that also emits the bf16 operational copy and
// applies the gradient-clip coefficient read from device memory (no host round trip).
//
// Data parallel (one process per GPU, NVLink peer memory): gradient reduce-scatter, Adam and the
// parameter all-gather are two kernels that talk to the peers directly:
//   dp_reduce_norm : the owner of a shard pulls that shard of every peer's fp32 gradient over
//                    NVLink, sums it, keeps the reduced shard locally and accumulates its squared
//                    norm (the clip needs the global norm before any weight moves);
//   dp_adam_push   : AdamW on the owner's fp32 master shard, then the new bf16 weights are stored
//                    straight into every peer's parameter buffer (the all-gather is the epilogue).
// Ordering across GPUs uses a flag barrier on a symmetric signal pad with a bounded spin that
// reports a timeout in a status word instead of hanging.
//
// This is the B200 form of the reference's ZeRO path: async reduce_scatter_tensor buckets
// (RPEG/runtime/workers/megatron_worker.py:1061-1067), FP32MasterAdamW.step
// (RPEG/runtime/optimizer_sharding.py:270), all_gather_into_tensor of the bf16 shards
// (megatron_worker.py:1262-1275) and the clip coefficient clamp(clip/(norm+1e-6), max=1)
// (megatron_worker.py:3231-3338).
#include "common.cuh"
#include "rpeg_kernels.h"

namespace rpeg {

__device__ __forceinline__ float clip_coef_from(const float* sumsq, int n_partials, float max_norm) {
  if (sumsq == nullptr || max_norm <= 0.f) return 1.f;
  float s = 0.f;
  for (int i = 0; i < n_partials; ++i) s += sumsq[i];
  return fminf(max_norm / (sqrtf(s) + 1e-6f), 1.f);
}

// p32/m/v fp32, grad fp32. w16 receives bf16(p32). step is 1-based.
__global__ void adamw_kernel(float* __restrict__ p32, float* __restrict__ m, float* __restrict__ v,
                             const float* __restrict__ grad, __nv_bfloat16* __restrict__ w16, long long n,
                             float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                             float grad_scale, const float* __restrict__ sumsq, int n_partials,
                             float max_norm) {
  const float gs = grad_scale * clip_coef_from(sumsq, n_partials, max_norm);
  const long long nv = n >> 2;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nv;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 p = reinterpret_cast<float4*>(p32)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    const float4 g = reinterpret_cast<const float4*>(grad)[i];
    float* pp = reinterpret_cast<float*>(&p);
    float* pm = reinterpret_cast<float*>(&mm);
    float* pv = reinterpret_cast<float*>(&vv);
    const float* pg = reinterpret_cast<const float*>(&g);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float gk = pg[k] * gs;
      pm[k] = beta1 * pm[k] + (1.f - beta1) * gk;
      pv[k] = beta2 * pv[k] + (1.f - beta2) * gk * gk;
      const float upd = (pm[k] / bc1) / (sqrtf(pv[k] / bc2) + eps);
      pp[k] = pp[k] * (1.f - lr * wd) - lr * upd;
    }
    reinterpret_cast<float4*>(p32)[i] = p;
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    uint2 o;
    o.x = pack_bf16x2(pp[0], pp[1]);
    o.y = pack_bf16x2(pp[2], pp[3]);
    reinterpret_cast<uint2*>(w16)[i] = o;
  }
}

// out[0] += sum x^2 (fp32 input)
__global__ void sumsq_kernel(const float* __restrict__ x, long long n, float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.f;
  const long long nv = n >> 2;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nv;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float4 a = reinterpret_cast<const float4*>(x)[i];
    s += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    s = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    s = warp_sum(s);
    if (threadIdx.x == 0) atomicAdd(out, s);
  }
}

struct PeerPtrs {
  void* p[RPEG_MAX_PEERS];
};

// Flag barrier over a symmetric signal pad. pad layout per rank: uint32 flag[RPEG_MAX_PEERS] at
// word offset `slot*RPEG_MAX_PEERS`. Rank r stores `epoch` into flag[r] of every peer, then waits
// until every flag in its own pad reached `epoch`. Optionally publishes one float per rank
// (payload area, word offset 1024 + slot*RPEG_MAX_PEERS) before the flag, e.g. a partial norm.
// The wait gives up after `timeout_ns` and records RPEG_ERR_FLAG_TIMEOUT in `status`.
__global__ void flag_barrier_kernel(PeerPtrs pads, int rank, int world, int slot, unsigned epoch,
                                    const float* __restrict__ payload_in, float* __restrict__ payload_out,
                                    unsigned long long timeout_ns, int* status) {
  const int t = threadIdx.x;
  if (t < world) {
    unsigned* peer = static_cast<unsigned*>(pads.p[t]);
    if (payload_in != nullptr) {
      reinterpret_cast<float*>(peer)[1024 + slot * RPEG_MAX_PEERS + rank] = payload_in[0];
    }
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peer + slot * RPEG_MAX_PEERS + rank), "r"(epoch)
                 : "memory");
    const unsigned* mine = static_cast<const unsigned*>(pads.p[rank]) + slot * RPEG_MAX_PEERS + t;
    unsigned seen = 0;
    const uint64_t t0 = global_timer_ns();
    for (;;) {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
      if (static_cast<int>(seen - epoch) >= 0) break;
      if (global_timer_ns() - t0 > timeout_ns) {
        record_error(status, RPEG_ERR_FLAG_TIMEOUT, 400 + slot, t);
        break;
      }
      __nanosleep(64);
    }
    if (payload_out != nullptr)
      payload_out[t] = reinterpret_cast<const volatile float*>(pads.p[rank])[1024 + slot * RPEG_MAX_PEERS + t];
  }
}

// Version words for pushed data (weights for generation ranks, rollout rows for training ranks). The pusher
// runs its copy kernels, then this kernel on the same stream: a system-scope fence followed by a release
// store of `version` into the word `word` of every destination's flag array. A consumer that sees the word
// has the data (reference: weight-version bookkeeping of RPEG/runtime/weight_versions.py:25-90, where a
// consumer of step k needs version max(0, k - 1 - tau)).
__global__ void publish_version_kernel(PeerPtrs flags, int n_dst, int word, unsigned version) {
  const int t = threadIdx.x;
  if (t < n_dst) {
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(static_cast<unsigned*>(flags.p[t]) + word), "r"(version)
                 : "memory");
  }
}

// result[0] = 1 when flags[0..n) all reached `min_version` within `timeout_ns`, else 0 (a poll that runs out is
// not an error: the host repeats it, so that no kernel ever waits longer than the caller's short bound).
__global__ void wait_flags_kernel(const unsigned* __restrict__ flags, int n, unsigned min_version,
                                  unsigned long long timeout_ns, int* __restrict__ result) {
  const int t = threadIdx.x;
  bool ok = true;
  if (t < n) {
    const uint64_t t0 = global_timer_ns();
    for (;;) {
      unsigned seen;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flags + t) : "memory");
      if (static_cast<int>(seen - min_version) >= 0) break;
      if (global_timer_ns() - t0 > timeout_ns) { ok = false; break; }
      __nanosleep(1000);
    }
  }
  ok = __all_sync(0xffffffffu, ok);
  if (t == 0) result[0] = ok ? 1 : 0;
}

// reduced[i] = scale * sum_p grads[p][shard_off + i], i in [0, shard_n); sumsq[0] += sum reduced^2.
// Loads from peer memory are latency bound per request, so every thread keeps 2 x world independent 16-byte loads
// in flight (all peers of two vectors) before it adds anything up. With a multicast mapping of the gradient
// buffers (`mc` != nullptr) one multimem.ld_reduce per vector lets NVSwitch add the ranks' copies instead: the
// owner then receives its shard once, not once per peer.
__global__ void __launch_bounds__(256)
dp_reduce_norm_kernel(PeerPtrs grads, const float* __restrict__ mc, int world, long long shard_off, long long shard_n,
                      float scale, float* __restrict__ reduced, float* __restrict__ sumsq) {
  __shared__ float red[32];
  float s = 0.f;
  const long long nv = shard_n >> 2;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < nv; i0 += 2 * stride) {
    const long long i1 = i0 + stride;
    const bool two = i1 < nv;
    float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0;
    if (mc != nullptr) {
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                   : "=f"(a0.x), "=f"(a0.y), "=f"(a0.z), "=f"(a0.w)
                   : "l"(reinterpret_cast<const float4*>(mc + shard_off) + i0)
                   : "memory");
      if (two)
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                     : "=f"(a1.x), "=f"(a1.y), "=f"(a1.z), "=f"(a1.w)
                     : "l"(reinterpret_cast<const float4*>(mc + shard_off) + i1)
                     : "memory");
    } else {
      float4 g0[RPEG_MAX_PEERS], g1[RPEG_MAX_PEERS];
#pragma unroll
      for (int p = 0; p < RPEG_MAX_PEERS; ++p) {
        if (p < world) {
          const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(grads.p[p]) + shard_off);
          g0[p] = src[i0];
          if (two) g1[p] = src[i1];
        }
      }
#pragma unroll
      for (int p = 0; p < RPEG_MAX_PEERS; ++p) {
        if (p < world) {
          a0.x += g0[p].x; a0.y += g0[p].y; a0.z += g0[p].z; a0.w += g0[p].w;
          if (two) { a1.x += g1[p].x; a1.y += g1[p].y; a1.z += g1[p].z; a1.w += g1[p].w; }
        }
      }
    }
    a0.x *= scale; a0.y *= scale; a0.z *= scale; a0.w *= scale;
    reinterpret_cast<float4*>(reduced)[i0] = a0;
    s += a0.x * a0.x + a0.y * a0.y + a0.z * a0.z + a0.w * a0.w;
    if (two) {
      a1.x *= scale; a1.y *= scale; a1.z *= scale; a1.w *= scale;
      reinterpret_cast<float4*>(reduced)[i1] = a1;
      s += a1.x * a1.x + a1.y * a1.y + a1.z * a1.z + a1.w * a1.w;
    }
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    s = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    s = warp_sum(s);
    if (threadIdx.x == 0) atomicAdd(sumsq, s);
  }
}

// AdamW on the local shard, then the bf16 result goes to every peer's parameter buffer.
__global__ void dp_adam_push_kernel(float* __restrict__ p32, float* __restrict__ m, float* __restrict__ v,
                                    const float* __restrict__ reduced, PeerPtrs params, int world,
                                    long long shard_off, long long shard_n, float lr, float beta1, float beta2,
                                    float eps, float wd, float bc1, float bc2, const float* __restrict__ sumsq,
                                    int n_partials, float max_norm) {
  const float gs = clip_coef_from(sumsq, n_partials, max_norm);
  const long long nv = shard_n >> 2;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nv;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 p = reinterpret_cast<float4*>(p32)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    const float4 g = reinterpret_cast<const float4*>(reduced)[i];
    float* pp = reinterpret_cast<float*>(&p);
    float* pm = reinterpret_cast<float*>(&mm);
    float* pv = reinterpret_cast<float*>(&vv);
    const float* pg = reinterpret_cast<const float*>(&g);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float gk = pg[k] * gs;
      pm[k] = beta1 * pm[k] + (1.f - beta1) * gk;
      pv[k] = beta2 * pv[k] + (1.f - beta2) * gk * gk;
      const float upd = (pm[k] / bc1) / (sqrtf(pv[k] / bc2) + eps);
      pp[k] = pp[k] * (1.f - lr * wd) - lr * upd;
    }
    reinterpret_cast<float4*>(p32)[i] = p;
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    uint2 o;
    o.x = pack_bf16x2(pp[0], pp[1]);
    o.y = pack_bf16x2(pp[2], pp[3]);
    for (int q = 0; q < world; ++q)
      reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(params.p[q]) + shard_off)[i] = o;
  }
}

// dst[i] = src[i] for 16-byte vectors; used for peer-memory pulls/pushes of weight shards.
__global__ void copy16_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long nvec) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    dst[i] = src[i];
}

}  // namespace rpeg

using namespace rpeg;
#define STREAM(s) reinterpret_cast<cudaStream_t>(s)
#define LAUNCH_OK() (cudaGetLastError() == cudaSuccess ? 0 : -21)
static inline unsigned sat_grid(long long work_items, int block) {
  long long g = (work_items + block - 1) / block;
  const long long cap = 148 * 8;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return static_cast<unsigned>(g);
}
static PeerPtrs make_peers(void* const* ptrs, int world) {
  PeerPtrs pp;
  for (int i = 0; i < RPEG_MAX_PEERS; ++i) pp.p[i] = i < world ? ptrs[i] : nullptr;
  return pp;
}

extern "C" int rpeg_adamw(float* p32, float* m, float* v, const float* grad, void* w16, long long n, float lr,
                          float beta1, float beta2, float eps, float wd, int step, float grad_scale,
                          const float* sumsq, int n_partials, float max_norm, void* stream) {
  if (n <= 0) return 0;
  if (n & 3) return -2;
  const float bc1 = 1.f - powf(beta1, static_cast<float>(step));
  const float bc2 = 1.f - powf(beta2, static_cast<float>(step));
  adamw_kernel<<<sat_grid(n >> 2, 256), 256, 0, STREAM(stream)>>>(p32, m, v, grad,
                                                                static_cast<__nv_bfloat16*>(w16), n, lr, beta1,
                                                                beta2, eps, wd, bc1, bc2, grad_scale, sumsq,
                                                                n_partials, max_norm);
  return LAUNCH_OK();
}

extern "C" int rpeg_sumsq(const float* x, long long n, float* out, void* stream) {
  if (n <= 0) return 0;
  if (n & 3) return -2;
  sumsq_kernel<<<sat_grid(n >> 2, 256), 256, 0, STREAM(stream)>>>(x, n, out);
  return LAUNCH_OK();
}

extern "C" int rpeg_flag_barrier(void* const* pads, int rank, int world, int slot, unsigned epoch,
                                 const float* payload_in, float* payload_out, unsigned long long timeout_ns,
                                 int* status, void* stream) {
  if (world < 1 || world > RPEG_MAX_PEERS || slot < 0 || slot >= 64) return -2;
  flag_barrier_kernel<<<1, 32, 0, STREAM(stream)>>>(make_peers(pads, world), rank, world, slot, epoch,
                                                   payload_in, payload_out, timeout_ns, status);
  return LAUNCH_OK();
}

extern "C" int rpeg_publish_version(void* const* flag_arrays, int n_dst, int word, unsigned version, void* stream) {
  if (n_dst < 1 || n_dst > RPEG_MAX_PEERS || word < 0) return -2;
  publish_version_kernel<<<1, 32, 0, STREAM(stream)>>>(make_peers(flag_arrays, n_dst), n_dst, word, version);
  return LAUNCH_OK();
}

extern "C" int rpeg_wait_flags(const unsigned* flags, int n, unsigned min_version, unsigned long long timeout_ns,
                               int* result, void* stream) {
  if (n < 1 || n > 32 || result == nullptr) return -2;
  wait_flags_kernel<<<1, 32, 0, STREAM(stream)>>>(flags, n, min_version, timeout_ns, result);
  return LAUNCH_OK();
}

static int reduce_norm_impl(void* const* grads, const float* mc, int world, long long shard_off, long long shard_n,
                            float scale, float* reduced, float* sumsq, void* stream) {
  if (world < 1 || world > RPEG_MAX_PEERS) return -2;
  if ((shard_off | shard_n) & 3) return -3;
  if (shard_n <= 0) return 0;
  dp_reduce_norm_kernel<<<sat_grid(shard_n >> 3, 256), 256, 0, STREAM(stream)>>>(make_peers(grads, world), mc, world,
                                                                               shard_off, shard_n, scale,
                                                                               reduced, sumsq);
  return LAUNCH_OK();
}

extern "C" int rpeg_dp_reduce_norm(void* const* grads, int world, long long shard_off, long long shard_n,
                                   float scale, float* reduced, float* sumsq, void* stream) {
  return reduce_norm_impl(grads, nullptr, world, shard_off, shard_n, scale, reduced, sumsq, stream);
}

// The same reduction through an NVLink multicast mapping of the gradient buffers (`mc` = multicast address of the
// buffers' base): NVSwitch adds the ranks' copies, the owner receives the sum.
extern "C" int rpeg_dp_reduce_norm_mc(const float* mc, int world, long long shard_off, long long shard_n, float scale,
                                      float* reduced, float* sumsq, void* stream) {
  if (mc == nullptr) return -4;
  void* none[RPEG_MAX_PEERS] = {nullptr};
  return reduce_norm_impl(none, mc, world, shard_off, shard_n, scale, reduced, sumsq, stream);
}

extern "C" int rpeg_dp_adam_push(float* p32, float* m, float* v, const float* reduced, void* const* params,
                                 int world, long long shard_off, long long shard_n, float lr, float beta1,
                                 float beta2, float eps, float wd, int step, const float* sumsq, int n_partials,
                                 float max_norm, void* stream) {
  if (world < 1 || world > RPEG_MAX_PEERS) return -2;
  if ((shard_off | shard_n) & 3) return -3;
  if (shard_n <= 0) return 0;
  const float bc1 = 1.f - powf(beta1, static_cast<float>(step));
  const float bc2 = 1.f - powf(beta2, static_cast<float>(step));
  dp_adam_push_kernel<<<sat_grid(shard_n >> 2, 256), 256, 0, STREAM(stream)>>>(
      p32, m, v, reduced, make_peers(params, world), world, shard_off, shard_n, lr, beta1, beta2, eps, wd, bc1,
      bc2, sumsq, n_partials, max_norm);
  return LAUNCH_OK();
}

// Strided rectangle copy (rows x row_bytes, pitches in bytes), source or destination may be peer memory.
// 16-byte vectors when pitches, row length and both bases allow it, else 2-byte elements.
template <typename V>
__global__ void copy2d_kernel(const uint8_t* __restrict__ src, long long src_pitch, uint8_t* __restrict__ dst,
                              long long dst_pitch, long long rows, long long vec_per_row) {
  const long long total = rows * vec_per_row;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vec_per_row, c = i % vec_per_row;
    reinterpret_cast<V*>(dst + r * dst_pitch)[c] = reinterpret_cast<const V*>(src + r * src_pitch)[c];
  }
}

extern "C" int rpeg_copy2d(const void* src, long long src_pitch, void* dst, long long dst_pitch, long long rows,
                           long long row_bytes, void* stream) {
  if (rows <= 0 || row_bytes <= 0) return 0;
  if ((row_bytes & 1) || (src_pitch & 1) || (dst_pitch & 1)) return -2;
  const uintptr_t all = reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst) | static_cast<uintptr_t>(src_pitch) |
                        static_cast<uintptr_t>(dst_pitch) | static_cast<uintptr_t>(row_bytes);
  if ((all & 15) == 0) {
    const long long v = row_bytes >> 4;
    copy2d_kernel<uint4><<<sat_grid(rows * v, 256), 256, 0, STREAM(stream)>>>(static_cast<const uint8_t*>(src), src_pitch,
                                                                            static_cast<uint8_t*>(dst), dst_pitch, rows, v);
  } else {
    const long long v = row_bytes >> 1;
    copy2d_kernel<uint16_t><<<sat_grid(rows * v, 256), 256, 0, STREAM(stream)>>>(static_cast<const uint8_t*>(src), src_pitch,
                                                                               static_cast<uint8_t*>(dst), dst_pitch, rows, v);
  }
  return LAUNCH_OK();
}

// Rows of a local [n, row_bytes] buffer go to the rank that owns their GLOBAL index (owner = idx / rows_per_rank,
// slot = idx % rows_per_rank) inside symmetric destination buffers: the hand-over of rollout rows (tokens,
// log-probs, values, rewards) between vertices whose data-parallel layouts differ. One warp per row.
__global__ void scatter_rows_by_index_kernel(const uint8_t* __restrict__ src, long long n, long long row_bytes,
                                             const long long* __restrict__ global_idx, long long rows_per_rank, PeerPtrs dst,
                                             int world) {
  const long long w = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (w >= n) return;
  const int lane = threadIdx.x & 31;
  const long long g = global_idx[w];
  const long long owner = g / rows_per_rank;
  if (g < 0 || owner >= world) return;
  uint8_t* out = static_cast<uint8_t*>(dst.p[owner]) + (g - owner * rows_per_rank) * row_bytes;
  const uint8_t* in = src + w * row_bytes;
  if (((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(in) | static_cast<uintptr_t>(row_bytes)) & 15) == 0) {
    for (long long i = lane; i < (row_bytes >> 4); i += 32) reinterpret_cast<uint4*>(out)[i] = reinterpret_cast<const uint4*>(in)[i];
  } else {
    for (long long i = lane; i < (row_bytes >> 2); i += 32) reinterpret_cast<uint32_t*>(out)[i] = reinterpret_cast<const uint32_t*>(in)[i];
  }
}

extern "C" int rpeg_scatter_rows_by_index(const void* src, long long n, long long row_bytes, const long long* global_idx,
                                          long long rows_per_rank, void* const* dst, int world, void* stream) {
  if (world < 1 || world > RPEG_MAX_PEERS || rows_per_rank <= 0) return -2;
  if (row_bytes <= 0 || (row_bytes & 3)) return -3;
  if (n <= 0) return 0;
  scatter_rows_by_index_kernel<<<static_cast<unsigned>((n * 32 + 255) / 256), 256, 0, STREAM(stream)>>>(
      static_cast<const uint8_t*>(src), n, row_bytes, global_idx, rows_per_rank, make_peers(dst, world), world);
  return LAUNCH_OK();
}

extern "C" int rpeg_copy16(const void* src, void* dst, long long nbytes, void* stream) {
  if (nbytes <= 0) return 0;
  if ((nbytes & 15) || (reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15)) return -2;
  copy16_kernel<<<sat_grid(nbytes >> 4, 256), 256, 0, STREAM(stream)>>>(static_cast<const uint4*>(src),
                                                                       static_cast<uint4*>(dst), nbytes >> 4);
  return LAUNCH_OK();
}
