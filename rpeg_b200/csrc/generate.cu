// Device-side bookkeeping of the decode loop, so a whole generation step (layers, LM head,
// sampling, state advance) replays as one CUDA graph with no host decision in between.
//
// Slot state (arrays of length n_slots, all on the device):
//   token[s]      next input token            pos[s]       its position (= tokens already cached)
//   seq_len[s]    keys visible to attention   active[s]    1 while the row is generating
//   gen_count[s]  tokens generated so far     forced_len[s] > 0: emit EOS as token number forced_len
//   out_tok/out_lp [s, max_new]               generated ids and their log-probs (the PPO old_logps)
//
// The reference keeps this state in Python per generation call and compacts KV rows on the host
// side after every EOS (RPEG/runtime/workers/megatron_worker.py:2463-2598).
#include "common.cuh"
#include "rpeg_kernels.h"

namespace rpeg {

// Before sampling: forced[s] = eos when the next token must be EOS (synthetic length control or
// the length cap), else -1.
__global__ void decode_prepare_kernel(const int* __restrict__ active, const int* __restrict__ gen_count,
                                      const int* __restrict__ forced_len, int* __restrict__ forced, int n_slots,
                                      int eos) {
  griddep_launch();
  griddep_wait();   // may have been scheduled under the previous kernel's tail: nothing is read or written before this
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= n_slots) return;
  int f = -1;
  if (active[s] && forced_len != nullptr && forced_len[s] > 0 && gen_count[s] + 1 >= forced_len[s]) f = eos;
  forced[s] = f;
}

// After sampling: record the token, retire rows that hit EOS or the cap, advance the others.
__global__ void decode_advance_kernel(const int* __restrict__ sampled, const float* __restrict__ sampled_lp,
                                      int* __restrict__ token, int* __restrict__ pos, int* __restrict__ seq_len,
                                      int* __restrict__ active, int* __restrict__ gen_count,
                                      int* __restrict__ out_tok, float* __restrict__ out_lp, int n_slots,
                                      int max_new, int eos, int* __restrict__ n_finished,
                                      unsigned long long* __restrict__ step_counter) {
  griddep_launch();
  griddep_wait();   // may have been scheduled under the previous kernel's tail: nothing is read or written before this
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s == 0 && step_counter != nullptr) step_counter[0] += 1;
  if (s >= n_slots || !active[s]) return;
  const int t = sampled[s];
  const int g = gen_count[s];
  out_tok[static_cast<size_t>(s) * max_new + g] = t;
  out_lp[static_cast<size_t>(s) * max_new + g] = sampled_lp[s];
  gen_count[s] = g + 1;
  if (t == eos || g + 1 >= max_new) {
    active[s] = 0;
    seq_len[s] = 0;  // attention of a retired slot reads nothing
    atomicAdd(n_finished, 1);
  } else {
    token[s] = t;
    pos[s] += 1;
    seq_len[s] += 1;
  }
}

// out[i, :] = x[rows[i], :]   (bf16 rows, 16-byte vectors)
__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ rows,
                                   __nv_bfloat16* __restrict__ out, int n, int d) {
  const int dv = d >> 3;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<long long>(n) * dv) return;
  const int i = static_cast<int>(idx / dv), j = static_cast<int>(idx % dv);
  reinterpret_cast<uint4*>(out + static_cast<size_t>(i) * d)[j] =
      reinterpret_cast<const uint4*>(x + static_cast<size_t>(rows[i]) * d)[j];
}

// x[rows[i], :] += src[i, :]   (rows are unique, so no atomics)
__global__ void scatter_add_rows_kernel(__nv_bfloat16* __restrict__ x, const int* __restrict__ rows,
                                        const __nv_bfloat16* __restrict__ src, int n, int d, int overwrite) {
  const int dv = d >> 3;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<long long>(n) * dv) return;
  const int i = static_cast<int>(idx / dv), j = static_cast<int>(idx % dv);
  uint4* dst = reinterpret_cast<uint4*>(x + static_cast<size_t>(rows[i]) * d) + j;
  uint4 s = reinterpret_cast<const uint4*>(src + static_cast<size_t>(i) * d)[j];
  if (!overwrite) {
    uint4 o = *dst;
    uint32_t *po = reinterpret_cast<uint32_t*>(&o), *ps = reinterpret_cast<uint32_t*>(&s);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 a = unpack_bf16x2(po[k]), b = unpack_bf16x2(ps[k]);
      ps[k] = pack_bf16x2(a.x + b.x, a.y + b.y);
    }
  }
  *dst = s;
}

// Split-K partial sums -> bf16: out[m, n] = sum_s part[s, m, n]
__global__ void splitk_reduce_kernel(const float* __restrict__ part, __nv_bfloat16* __restrict__ out, int M, int N,
                                     int ldc, int splits) {
  griddep_launch();
  griddep_wait();   // may have been scheduled under the previous kernel's tail: nothing is read or written before this
  const int nv = N >> 2;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<long long>(M) * nv) return;
  const int m = static_cast<int>(idx / nv), j = static_cast<int>(idx % nv);
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s = 0; s < splits; ++s) {
    const float4 p = reinterpret_cast<const float4*>(part + (static_cast<size_t>(s) * M + m) * N)[j];
    a.x += p.x; a.y += p.y; a.z += p.z; a.w += p.w;
  }
  uint2 o;
  o.x = pack_bf16x2(a.x, a.y);
  o.y = pack_bf16x2(a.z, a.w);
  *reinterpret_cast<uint2*>(out + static_cast<size_t>(m) * ldc + j * 4) = o;
}

}  // namespace rpeg

using namespace rpeg;
#define STREAM(s) reinterpret_cast<cudaStream_t>(s)
#define LAUNCH_OK() (cudaGetLastError() == cudaSuccess ? 0 : -21)

extern "C" int rpeg_decode_prepare(const int* active, const int* gen_count, const int* forced_len, int* forced,
                                   int n_slots, int eos, void* stream) {
  if (n_slots <= 0) return 0;
  launch_pdl(decode_prepare_kernel, dim3((n_slots + 127) / 128), dim3(128), 0, STREAM(stream), active, gen_count, forced_len, forced,
                                                                         n_slots, eos);
  return LAUNCH_OK();
}

extern "C" int rpeg_decode_advance(const int* sampled, const float* sampled_lp, int* token, int* pos, int* seq_len,
                                   int* active, int* gen_count, int* out_tok, float* out_lp, int n_slots,
                                   int max_new, int eos, int* n_finished, unsigned long long* step_counter,
                                   void* stream) {
  if (n_slots <= 0) return 0;
  launch_pdl(decode_advance_kernel, dim3((n_slots + 127) / 128), dim3(128), 0, STREAM(stream), 
      sampled, sampled_lp, token, pos, seq_len, active, gen_count, out_tok, out_lp, n_slots, max_new, eos, n_finished,
      step_counter);
  return LAUNCH_OK();
}

extern "C" int rpeg_gather_rows(const void* x, const int* rows, void* out, int n, int d, void* stream) {
  if (d & 7) return -2;
  const long long total = static_cast<long long>(n) * (d >> 3);
  if (total <= 0) return 0;
  gather_rows_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, STREAM(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), rows, static_cast<__nv_bfloat16*>(out), n, d);
  return LAUNCH_OK();
}

extern "C" int rpeg_scatter_rows(void* x, const int* rows, const void* src, int n, int d, int overwrite,
                                 void* stream) {
  if (d & 7) return -2;
  const long long total = static_cast<long long>(n) * (d >> 3);
  if (total <= 0) return 0;
  scatter_add_rows_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, STREAM(stream)>>>(
      static_cast<__nv_bfloat16*>(x), rows, static_cast<const __nv_bfloat16*>(src), n, d, overwrite);
  return LAUNCH_OK();
}

extern "C" int rpeg_splitk_reduce(const float* part, void* out, int M, int N, int ldc, int splits, void* stream) {
  if ((N & 3) || (ldc & 3)) return -2;
  const long long total = static_cast<long long>(M) * (N >> 2);
  if (total <= 0) return 0;
  launch_pdl(splitk_reduce_kernel, dim3(static_cast<unsigned>((total + 255) / 256)), dim3(256), 0, STREAM(stream), 
      part, static_cast<__nv_bfloat16*>(out), M, N, ldc, splits);
  return LAUNCH_OK();
}

// Switch programmatic dependent launches on or off for the kernels launched from now on (a CUDA graph keeps what was
// in force while it was captured). The environment's RPEG_PDL=0 wins.
extern "C" void rpeg_set_pdl(int on) {
  pdl_enabled();
  int& v = pdl_state();
  if (v != 2) v = on ? 1 : 0;
}

