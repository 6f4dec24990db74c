// RMSNorm (+ fused residual add) forward/backward, RoPE (rotate-half, in place) and SwiGLU
// forward/backward for sm_100a. All are HBM-bound row kernels: 16-byte vector accesses, one warp
// per token row, fp32 math, bf16 storage.
//
// The reference gets these from TransformerEngine / apex / ATen through megatron-core
// (RPEG/runtime/workers/megatron_worker.py:683 normalization, :686 activation; the rotary
// embedding is Megatron's) and measures them in calibrate.py:744-895.
#include "common.cuh"
#include "rpeg_kernels.h"

namespace rpeg {

constexpr int ROW_WARPS = 4;

// y = (x [+ res]) * rstd * w ; optionally writes h = x + res (the new residual stream).
__global__ void __launch_bounds__(ROW_WARPS * 32)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ h_out,
                   __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out, int T, int d, float eps) {
  const int row = blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
  if (row >= T) return;
  const int lane = threadIdx.x & 31;
  const int nvec = d >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * d);
  const uint4* rr = res ? reinterpret_cast<const uint4*>(res + static_cast<size_t>(row) * d) : nullptr;
  uint4* hr = h_out ? reinterpret_cast<uint4*>(h_out + static_cast<size_t>(row) * d) : nullptr;
  float ss = 0.f;
  for (int i = lane; i < nvec; i += 32) {
    uint4 v = xr[i];
    uint32_t* pv = reinterpret_cast<uint32_t*>(&v);
    if (rr) {
      uint4 r = rr[i];
      const uint32_t* pr = reinterpret_cast<const uint32_t*>(&r);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float2 a = unpack_bf16x2(pv[k]), b = unpack_bf16x2(pr[k]);
        pv[k] = pack_bf16x2(a.x + b.x, a.y + b.y);
      }
      if (hr) hr[i] = v;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 a = unpack_bf16x2(pv[k]);
      ss += a.x * a.x + a.y * a.y;
    }
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / static_cast<float>(d) + eps);
  if (lane == 0 && rstd_out) rstd_out[row] = rstd;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* yr = reinterpret_cast<uint4*>(y + static_cast<size_t>(row) * d);
  // Second pass re-reads the row (L1/L2 resident) rather than holding d/32 values per lane.
  const uint4* src = (rr && hr) ? reinterpret_cast<const uint4*>(hr) : xr;
  for (int i = lane; i < nvec; i += 32) {
    uint4 v = src[i];
    uint32_t* pv = reinterpret_cast<uint32_t*>(&v);
    if (rr && !hr) {
      uint4 r = rr[i];
      const uint32_t* pr = reinterpret_cast<const uint32_t*>(&r);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float2 a = unpack_bf16x2(pv[k]), b = unpack_bf16x2(pr[k]);
        pv[k] = pack_bf16x2(a.x + b.x, a.y + b.y);
      }
    }
    uint4 wv = wr[i];
    const uint32_t* pw = reinterpret_cast<const uint32_t*>(&wv);
    uint4 o;
    uint32_t* po = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 a = unpack_bf16x2(pv[k]), b = unpack_bf16x2(pw[k]);
      po[k] = pack_bf16x2(a.x * rstd * b.x, a.y * rstd * b.y);
    }
    yr[i] = o;
  }
}

// dx = rstd * (dy*w) - x * rstd^3/d * sum(dy*w*x) [+ dres_in];  dw += sum_rows dy * x * rstd.
// Each CTA walks `rows_per_cta` rows; lanes keep their dw columns in shared memory and flush with
// one atomicAdd per column per CTA.
__global__ void __launch_bounds__(ROW_WARPS * 32)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                   const __nv_bfloat16* __restrict__ dres_in, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dw, int T, int d, int rows_per_cta) {
  extern __shared__ float dw_sm[];  // [d]
  for (int i = threadIdx.x; i < d; i += blockDim.x) dw_sm[i] = 0.f;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = d >> 3;
  const int row0 = blockIdx.x * rows_per_cta;
  const int row1 = min(T, row0 + rows_per_cta);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  for (int row = row0 + warp; row < row1; row += ROW_WARPS) {
    const uint4* dyr = reinterpret_cast<const uint4*>(dy + static_cast<size_t>(row) * d);
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * d);
    const float rs = rstd[row];
    float dot = 0.f;
    for (int i = lane; i < nvec; i += 32) {
      uint4 a = dyr[i], b = xr[i], c = wr[i];
      const uint32_t *pa = reinterpret_cast<const uint32_t*>(&a), *pb = reinterpret_cast<const uint32_t*>(&b),
                     *pc = reinterpret_cast<const uint32_t*>(&c);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float2 g = unpack_bf16x2(pa[k]), xv = unpack_bf16x2(pb[k]), wv = unpack_bf16x2(pc[k]);
        dot += g.x * wv.x * xv.x + g.y * wv.y * xv.y;
      }
    }
    dot = warp_sum(dot);
    const float coef = dot * rs * rs * rs / static_cast<float>(d);
    const uint4* drr = dres_in ? reinterpret_cast<const uint4*>(dres_in + static_cast<size_t>(row) * d) : nullptr;
    uint4* dxr = reinterpret_cast<uint4*>(dx + static_cast<size_t>(row) * d);
    for (int i = lane; i < nvec; i += 32) {
      uint4 a = dyr[i], b = xr[i], c = wr[i];
      const uint32_t *pa = reinterpret_cast<const uint32_t*>(&a), *pb = reinterpret_cast<const uint32_t*>(&b),
                     *pc = reinterpret_cast<const uint32_t*>(&c);
      uint4 r = make_uint4(0, 0, 0, 0);
      if (drr) r = drr[i];
      const uint32_t* pr = reinterpret_cast<const uint32_t*>(&r);
      uint4 o;
      uint32_t* po = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float2 g = unpack_bf16x2(pa[k]), xv = unpack_bf16x2(pb[k]), wv = unpack_bf16x2(pc[k]);
        float2 rr = drr ? unpack_bf16x2(pr[k]) : make_float2(0.f, 0.f);
        const float o0 = rs * g.x * wv.x - xv.x * coef + rr.x;
        const float o1 = rs * g.y * wv.y - xv.y * coef + rr.y;
        po[k] = pack_bf16x2(o0, o1);
        atomicAdd(&dw_sm[i * 8 + 2 * k], g.x * xv.x * rs);
        atomicAdd(&dw_sm[i * 8 + 2 * k + 1], g.y * xv.y * rs);
      }
      dxr[i] = o;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < d; i += blockDim.x) atomicAdd(&dw[i], dw_sm[i]);
}

// Backward with fixed column ownership: 256 threads, thread t owns the 16-byte vectors t, t+256, ... of
// every row its CTA walks, so the dw partial sums stay in registers for the whole kernel (one global
// atomicAdd per column per CTA at the end) and the only per-row communication is the block-wide sum
// of dy*w*x. The next row's operands are loaded before the current row's reduction completes.
template <int NV>
__global__ void __launch_bounds__(256)
rmsnorm_bwd_row_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                       const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                       const __nv_bfloat16* __restrict__ dres_in, __nv_bfloat16* __restrict__ dx,
                       float* __restrict__ dw, int T, int d) {
  __shared__ float part[2][8];
  const int nvec = d >> 3;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float wf[NV][8], acc[NV][8];
  bool own[NV];
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = threadIdx.x + k * 256;
    own[k] = i < nvec;
#pragma unroll
    for (int e = 0; e < 8; ++e) { wf[k][e] = 0.f; acc[k][e] = 0.f; }
    if (own[k]) {
      const uint4 wv = reinterpret_cast<const uint4*>(w)[i];
      const uint32_t* pw = reinterpret_cast<const uint32_t*>(&wv);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = unpack_bf16x2(pw[e]);
        wf[k][2 * e] = f.x; wf[k][2 * e + 1] = f.y;
      }
    }
  }
  const float inv_d = 1.f / static_cast<float>(d);
  int it = 0;
  for (int row = blockIdx.x; row < T; row += gridDim.x, ++it) {
    uint4 a[NV], b[NV], r[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int i = threadIdx.x + k * 256;
      a[k] = b[k] = r[k] = make_uint4(0u, 0u, 0u, 0u);
      if (own[k]) {
        a[k] = reinterpret_cast<const uint4*>(dy + static_cast<size_t>(row) * d)[i];
        b[k] = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * d)[i];
        if (dres_in) r[k] = reinterpret_cast<const uint4*>(dres_in + static_cast<size_t>(row) * d)[i];
      }
    }
    const float rs = rstd[row];
    float g[NV][8], xv[NV][8];
    float dot = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const uint32_t *pa = reinterpret_cast<const uint32_t*>(&a[k]), *pb = reinterpret_cast<const uint32_t*>(&b[k]);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 ga = unpack_bf16x2(pa[e]), xb = unpack_bf16x2(pb[e]);
        g[k][2 * e] = ga.x; g[k][2 * e + 1] = ga.y; xv[k][2 * e] = xb.x; xv[k][2 * e + 1] = xb.y;
        dot += ga.x * wf[k][2 * e] * xb.x + ga.y * wf[k][2 * e + 1] * xb.y;
      }
    }
    dot = warp_sum(dot);
    float* slot = part[it & 1];
    if (lane == 0) slot[warp] = dot;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) tot += slot[k];
    const float coef = tot * rs * rs * rs * inv_d;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      if (!own[k]) continue;
      const uint32_t* pr = reinterpret_cast<const uint32_t*>(&r[k]);
      uint4 o;
      uint32_t* po = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 rr = unpack_bf16x2(pr[e]);
        const float o0 = rs * g[k][2 * e] * wf[k][2 * e] - xv[k][2 * e] * coef + rr.x;
        const float o1 = rs * g[k][2 * e + 1] * wf[k][2 * e + 1] - xv[k][2 * e + 1] * coef + rr.y;
        po[e] = pack_bf16x2(o0, o1);
        acc[k][2 * e] += g[k][2 * e] * xv[k][2 * e] * rs;
        acc[k][2 * e + 1] += g[k][2 * e + 1] * xv[k][2 * e + 1] * rs;
      }
      reinterpret_cast<uint4*>(dx + static_cast<size_t>(row) * d)[threadIdx.x + k * 256] = o;
    }
  }
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    if (!own[k]) continue;
    const int c0 = (threadIdx.x + k * 256) * 8;
#pragma unroll
    for (int e = 0; e < 8; ++e) atomicAdd(&dw[c0 + e], acc[k][e]);
  }
}

// Row-per-CTA variant: 256 threads keep the whole row in registers (NV 16-byte vectors per thread),
// so x and res are read once and nothing is re-read for the second pass. Used for d <= 8192.
template <int NV>
__global__ void __launch_bounds__(256)
rmsnorm_fwd_row_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                       const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ h_out,
                       __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out, int d, float eps) {
  griddep_launch();
  griddep_wait();   // may have been scheduled under the previous kernel's tail: nothing is read or written before this
  __shared__ float warp_ss[8];
  const int row = blockIdx.x;
  const int nvec = d >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * d);
  const uint4* rr = res ? reinterpret_cast<const uint4*>(res + static_cast<size_t>(row) * d) : nullptr;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4 v[NV], wv[NV];
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = threadIdx.x + k * 256;
    v[k] = make_uint4(0u, 0u, 0u, 0u);
    if (i < nvec) { v[k] = xr[i]; wv[k] = wr[i]; }
  }
  if (rr) {
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int i = threadIdx.x + k * 256;
      if (i < nvec) {
        const uint4 r = rr[i];
        const uint32_t* pr = reinterpret_cast<const uint32_t*>(&r);
        uint32_t* pv = reinterpret_cast<uint32_t*>(&v[k]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 a = unpack_bf16x2(pv[e]), b = unpack_bf16x2(pr[e]);
          pv[e] = pack_bf16x2(a.x + b.x, a.y + b.y);
        }
        if (h_out) reinterpret_cast<uint4*>(h_out + static_cast<size_t>(row) * d)[i] = v[k];
      }
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const uint32_t* pv = reinterpret_cast<const uint32_t*>(&v[k]);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 a = unpack_bf16x2(pv[e]);
      ss += a.x * a.x + a.y * a.y;
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) warp_ss[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) tot += warp_ss[k];
  const float rstd = rsqrtf(tot / static_cast<float>(d) + eps);
  if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
  uint4* yr = reinterpret_cast<uint4*>(y + static_cast<size_t>(row) * d);
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = threadIdx.x + k * 256;
    if (i < nvec) {
      const uint32_t* pv = reinterpret_cast<const uint32_t*>(&v[k]);
      const uint32_t* pw = reinterpret_cast<const uint32_t*>(&wv[k]);
      uint4 o;
      uint32_t* po = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 a = unpack_bf16x2(pv[e]), b = unpack_bf16x2(pw[e]);
        po[e] = pack_bf16x2(a.x * rstd * b.x, a.y * rstd * b.y);
      }
      yr[i] = o;
    }
  }
}

// Per-head RMSNorm ("QK-norm"): every (token, head) slice of width 128 inside a [T, ld] buffer at column
// col0 is normalised in place, y = x * rstd * w with one weight vector w[128] shared by all heads.
// One warp per (token, head); a lane owns 4 elements. rstd_out [T * nheads] keeps 1/rms for backward.
__global__ void __launch_bounds__(256)
headnorm_fwd_kernel(__nv_bfloat16* __restrict__ buf, int ld, int col0, int nheads, const __nv_bfloat16* __restrict__ w,
                    float* __restrict__ rstd_out, long long rows, float eps) {
  const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (wid >= rows) return;
  const int lane = threadIdx.x & 31;
  const long long t = wid / nheads;
  const int h = static_cast<int>(wid % nheads);
  __nv_bfloat16* p = buf + t * ld + col0 + h * 128 + lane * 4;
  const uint2 v = *reinterpret_cast<const uint2*>(p);
  const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y);
  const float ss = warp_sum(a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y);
  const float rstd = rsqrtf(ss * (1.f / 128.f) + eps);
  if (lane == 0 && rstd_out) rstd_out[wid] = rstd;
  const uint2 wv = *reinterpret_cast<const uint2*>(w + lane * 4);
  const float2 w0 = unpack_bf16x2(wv.x), w1 = unpack_bf16x2(wv.y);
  uint2 o;
  o.x = pack_bf16x2(a.x * rstd * w0.x, a.y * rstd * w0.y);
  o.y = pack_bf16x2(b.x * rstd * w1.x, b.y * rstd * w1.y);
  *reinterpret_cast<uint2*>(p) = o;
}

// Backward of the per-head norm, in place on the gradient buffer: dbuf holds dy on entry and dx on exit;
// x is the PRE-norm input in the same layout. dx = rstd * (w*dy - xhat * mean(w*dy*xhat)), dw += dy * xhat.
__global__ void __launch_bounds__(256)
headnorm_bwd_kernel(__nv_bfloat16* __restrict__ dbuf, int ldd, const __nv_bfloat16* __restrict__ x, int ldx, int col0,
                    int nheads, const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                    float* __restrict__ dw, long long rows) {
  __shared__ float dw_sm[128];
  if (threadIdx.x < 128) dw_sm[threadIdx.x] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const long long warps_total = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  const uint2 wv = *reinterpret_cast<const uint2*>(w + lane * 4);
  const float2 w0 = unpack_bf16x2(wv.x), w1 = unpack_bf16x2(wv.y);
  for (long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; wid < rows; wid += warps_total) {
    const long long t = wid / nheads;
    const int h = static_cast<int>(wid % nheads);
    const uint2 xv = *reinterpret_cast<const uint2*>(x + t * ldx + col0 + h * 128 + lane * 4);
    __nv_bfloat16* dp = dbuf + t * ldd + col0 + h * 128 + lane * 4;
    const uint2 dv = *reinterpret_cast<const uint2*>(dp);
    const float r = rstd[wid];
    const float2 x0 = unpack_bf16x2(xv.x), x1 = unpack_bf16x2(xv.y), d0 = unpack_bf16x2(dv.x), d1 = unpack_bf16x2(dv.y);
    const float xh[4] = {x0.x * r, x0.y * r, x1.x * r, x1.y * r};
    const float dy[4] = {d0.x, d0.y, d1.x, d1.y};
    const float wd[4] = {w0.x * dy[0], w0.y * dy[1], w1.x * dy[2], w1.y * dy[3]};
    const float m = warp_sum(wd[0] * xh[0] + wd[1] * xh[1] + wd[2] * xh[2] + wd[3] * xh[3]) * (1.f / 128.f);
    uint2 o;
    o.x = pack_bf16x2(r * (wd[0] - xh[0] * m), r * (wd[1] - xh[1] * m));
    o.y = pack_bf16x2(r * (wd[2] - xh[2] * m), r * (wd[3] - xh[3] * m));
    *reinterpret_cast<uint2*>(dp) = o;
#pragma unroll
    for (int k = 0; k < 4; ++k) acc[k] += dy[k] * xh[k];
  }
#pragma unroll
  for (int k = 0; k < 4; ++k) atomicAdd(&dw_sm[lane * 4 + k], acc[k]);
  __syncthreads();
  if (threadIdx.x < 128) atomicAdd(&dw[threadIdx.x], dw_sm[threadIdx.x]);
}

// ---- consumers of split-K partials (decode): x = sum_s parts[s] is formed while loading --------------
__device__ __forceinline__ void load_partials8(const float* __restrict__ parts, int splits, long long stride, size_t off,
                                               float (&v)[8]) {
#pragma unroll
  for (int e = 0; e < 8; ++e) v[e] = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float4 a = *reinterpret_cast<const float4*>(parts + s * stride + off);
    const float4 b = *reinterpret_cast<const float4*>(parts + s * stride + off + 4);
    v[0] += a.x; v[1] += a.y; v[2] += a.z; v[3] += a.w; v[4] += b.x; v[5] += b.y; v[6] += b.z; v[7] += b.w;
  }
}

// y = rmsnorm(sum_s parts[s] [+ res]) * w; h_out (optional) = the bf16 sum, i.e. the new residual stream.
template <int NV>
__global__ void __launch_bounds__(256)
rmsnorm_fwd_partials_kernel(const float* __restrict__ parts, int splits, long long stride,
                            const __nv_bfloat16* __restrict__ res, const __nv_bfloat16* __restrict__ w,
                            __nv_bfloat16* __restrict__ h_out, __nv_bfloat16* __restrict__ y, int d, float eps) {
  griddep_launch();
  griddep_wait();   // may have been scheduled under the previous kernel's tail: nothing is read or written before this
  __shared__ float warp_ss[8];
  const int row = blockIdx.x;
  const int nvec = d >> 3;
  float v[NV][8];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = threadIdx.x + k * 256;
#pragma unroll
    for (int e = 0; e < 8; ++e) v[k][e] = 0.f;
    if (i < nvec) {
      load_partials8(parts, splits, stride, static_cast<size_t>(row) * d + i * 8, v[k]);
      if (res) {
        const uint4 r = reinterpret_cast<const uint4*>(res + static_cast<size_t>(row) * d)[i];
        const uint32_t* pr = reinterpret_cast<const uint32_t*>(&r);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = unpack_bf16x2(pr[e]);
          v[k][2 * e] += f.x; v[k][2 * e + 1] += f.y;
        }
      }
      // the residual stream is kept in bf16: round here so the norm sees exactly what is stored
      uint4 hv;
      uint32_t* ph = reinterpret_cast<uint32_t*>(&hv);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        ph[e] = pack_bf16x2(v[k][2 * e], v[k][2 * e + 1]);
        const float2 f = unpack_bf16x2(ph[e]);
        v[k][2 * e] = f.x; v[k][2 * e + 1] = f.y;
        ss += f.x * f.x + f.y * f.y;
      }
      if (h_out) reinterpret_cast<uint4*>(h_out + static_cast<size_t>(row) * d)[i] = hv;
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) warp_ss[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) tot += warp_ss[k];
  const float rstd = rsqrtf(tot / static_cast<float>(d) + eps);
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = threadIdx.x + k * 256;
    if (i < nvec) {
      const uint4 wv = reinterpret_cast<const uint4*>(w)[i];
      const uint32_t* pw = reinterpret_cast<const uint32_t*>(&wv);
      uint4 o;
      uint32_t* po = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 b = unpack_bf16x2(pw[e]);
        po[e] = pack_bf16x2(v[k][2 * e] * rstd * b.x, v[k][2 * e + 1] * rstd * b.y);
      }
      reinterpret_cast<uint4*>(y + static_cast<size_t>(row) * d)[i] = o;
    }
  }
}

// out[t, j] = silu(g) * u with [g | u] = sum_s parts[s][t, :]
__global__ void swiglu_fwd_partials_kernel(const float* __restrict__ parts, int splits, long long stride,
                                           __nv_bfloat16* __restrict__ out, long long T, int f) {
  griddep_launch();
  griddep_wait();   // may have been scheduled under the previous kernel's tail: nothing is read or written before this
  const int fv = f >> 3;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= T * fv) return;
  const long long t = idx / fv;
  const int j = static_cast<int>(idx % fv) * 8;
  float g[8], u[8];
  load_partials8(parts, splits, stride, static_cast<size_t>(t) * 2 * f + j, g);
  load_partials8(parts, splits, stride, static_cast<size_t>(t) * 2 * f + f + j, u);
  uint4 o;
  uint32_t* po = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    // the unfused path rounds the GEMM output to bf16 before the activation; do the same
    const float2 gg = unpack_bf16x2(pack_bf16x2(g[2 * e], g[2 * e + 1])), uu = unpack_bf16x2(pack_bf16x2(u[2 * e], u[2 * e + 1]));
    po[e] = pack_bf16x2(gg.x / (1.f + __expf(-gg.x)) * uu.x, gg.y / (1.f + __expf(-gg.y)) * uu.y);
  }
  reinterpret_cast<uint4*>(out + t * f)[j >> 3] = o;
}

// RoPE, rotate-half pairing (i, i + hd/2), applied in place to `nheads` heads of width hd that sit
// at column offset `col0` of a [T, ld] bf16 buffer. cos/sin tables are fp32 [max_pos, hd/2].
// sign = +1 forward, -1 backward (the transpose of a rotation is the rotation by -angle).
__global__ void rope_kernel(__nv_bfloat16* __restrict__ buf, const int* __restrict__ pos,
                            const float* __restrict__ cos_t, const float* __restrict__ sin_t, int T, int ld,
                            int col0, int nheads, int hd, float sign) {
  const int half = hd >> 1;
  const int pairs_per_row = nheads * (half >> 1);  // each thread rotates 2 adjacent pairs
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<long long>(T) * pairs_per_row) return;
  const int t = static_cast<int>(idx / pairs_per_row);
  const int r = static_cast<int>(idx % pairs_per_row);
  const int head = r / (half >> 1);
  const int i = (r % (half >> 1)) * 2;
  const int p = pos[t];
  __nv_bfloat16* base = buf + static_cast<size_t>(t) * ld + col0 + head * hd;
  const float2 c = *reinterpret_cast<const float2*>(cos_t + static_cast<size_t>(p) * half + i);
  float2 s = *reinterpret_cast<const float2*>(sin_t + static_cast<size_t>(p) * half + i);
  s.x *= sign;
  s.y *= sign;
  uint32_t lo = *reinterpret_cast<uint32_t*>(base + i);
  uint32_t hi = *reinterpret_cast<uint32_t*>(base + i + half);
  const float2 a = unpack_bf16x2(lo), b = unpack_bf16x2(hi);
  lo = pack_bf16x2(a.x * c.x - b.x * s.x, a.y * c.y - b.y * s.y);
  hi = pack_bf16x2(b.x * c.x + a.x * s.x, b.y * c.y + a.y * s.y);
  *reinterpret_cast<uint32_t*>(base + i) = lo;
  *reinterpret_cast<uint32_t*>(base + i + half) = hi;
}

// out[t, j] = silu(gu[t, j]) * gu[t, f + j]
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                                  long long T, int f) {
  griddep_launch();   // a following decode GEMM may start its set-up and weight prefetch now
  const int fv = f >> 3;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= T * fv) return;
  const long long t = idx / fv;
  const int j = static_cast<int>(idx % fv);
  const uint4 g = reinterpret_cast<const uint4*>(gu + t * 2 * f)[j];
  const uint4 u = reinterpret_cast<const uint4*>(gu + t * 2 * f + f)[j];
  const uint32_t *pg = reinterpret_cast<const uint32_t*>(&g), *pu = reinterpret_cast<const uint32_t*>(&u);
  uint4 o;
  uint32_t* po = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    float2 a = unpack_bf16x2(pg[k]), b = unpack_bf16x2(pu[k]);
    const float s0 = a.x / (1.f + __expf(-a.x)), s1 = a.y / (1.f + __expf(-a.y));
    po[k] = pack_bf16x2(s0 * b.x, s1 * b.y);
  }
  reinterpret_cast<uint4*>(out + t * f)[j] = o;
}

// dgu[t, j] = dout * u * d silu(g);  dgu[t, f + j] = dout * silu(g)
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dout,
                                  __nv_bfloat16* __restrict__ dgu, long long T, int f) {
  const int fv = f >> 3;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= T * fv) return;
  const long long t = idx / fv;
  const int j = static_cast<int>(idx % fv);
  const uint4 g = reinterpret_cast<const uint4*>(gu + t * 2 * f)[j];
  const uint4 u = reinterpret_cast<const uint4*>(gu + t * 2 * f + f)[j];
  const uint4 d = reinterpret_cast<const uint4*>(dout + t * f)[j];
  const uint32_t *pg = reinterpret_cast<const uint32_t*>(&g), *pu = reinterpret_cast<const uint32_t*>(&u),
                 *pd = reinterpret_cast<const uint32_t*>(&d);
  uint4 og, ou;
  uint32_t *pog = reinterpret_cast<uint32_t*>(&og), *pou = reinterpret_cast<uint32_t*>(&ou);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    float2 a = unpack_bf16x2(pg[k]), b = unpack_bf16x2(pu[k]), c = unpack_bf16x2(pd[k]);
    const float sg0 = 1.f / (1.f + __expf(-a.x)), sg1 = 1.f / (1.f + __expf(-a.y));
    const float si0 = a.x * sg0, si1 = a.y * sg1;
    pog[k] = pack_bf16x2(c.x * b.x * (sg0 + si0 * (1.f - sg0)), c.y * b.y * (sg1 + si1 * (1.f - sg1)));
    pou[k] = pack_bf16x2(c.x * si0, c.y * si1);
  }
  reinterpret_cast<uint4*>(dgu + t * 2 * f)[j] = og;
  reinterpret_cast<uint4*>(dgu + t * 2 * f + f)[j] = ou;
}

// out[i] = a[i] + b[i] (bf16), 8 elements per thread.
__global__ void add_bf16_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                __nv_bfloat16* __restrict__ out, long long nvec) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= nvec) return;
  const uint4 x = reinterpret_cast<const uint4*>(a)[i], y = reinterpret_cast<const uint4*>(b)[i];
  const uint32_t *px = reinterpret_cast<const uint32_t*>(&x), *py = reinterpret_cast<const uint32_t*>(&y);
  uint4 o;
  uint32_t* po = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    float2 p = unpack_bf16x2(px[k]), q = unpack_bf16x2(py[k]);
    po[k] = pack_bf16x2(p.x + q.x, p.y + q.y);
  }
  reinterpret_cast<uint4*>(out)[i] = o;
}

// Row gather of an embedding table and its backward scatter-add into an fp32 gradient.
__global__ void embed_fwd_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                 __nv_bfloat16* __restrict__ out, int T, int d) {
  griddep_launch();
  griddep_wait();   // may have been scheduled under the previous kernel's tail: nothing is read or written before this
  const int dv = d >> 3;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<long long>(T) * dv) return;
  const int t = static_cast<int>(idx / dv), j = static_cast<int>(idx % dv);
  reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * d)[j] =
      reinterpret_cast<const uint4*>(table + static_cast<size_t>(ids[t]) * d)[j];
}
__global__ void embed_bwd_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ dout,
                                 float* __restrict__ dtable, int T, int d) {
  const int dv = d >> 1;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<long long>(T) * dv) return;
  const int t = static_cast<int>(idx / dv), j = static_cast<int>(idx % dv);
  const float2 g = unpack_bf16x2(reinterpret_cast<const uint32_t*>(dout + static_cast<size_t>(t) * d)[j]);
  float* dst = dtable + static_cast<size_t>(ids[t]) * d + 2 * j;
  atomicAdd(dst, g.x);
  atomicAdd(dst + 1, g.y);
}

}  // namespace rpeg

using namespace rpeg;
#define STREAM(s) reinterpret_cast<cudaStream_t>(s)
#define LAUNCH_OK() (cudaGetLastError() == cudaSuccess ? 0 : -21)

extern "C" int rpeg_rmsnorm_fwd(const void* x, const void* res, const void* w, void* h_out, void* y,
                                float* rstd, int T, int d, float eps, void* stream) {
  if (d & 7) return -2;
  if (T <= 0) return 0;
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* rp = static_cast<const __nv_bfloat16*>(res);
  const __nv_bfloat16* wp = static_cast<const __nv_bfloat16*>(w);
  __nv_bfloat16* hp = static_cast<__nv_bfloat16*>(h_out);
  __nv_bfloat16* yp = static_cast<__nv_bfloat16*>(y);
  const int nv = ((d >> 3) + 255) / 256;
  if (nv == 1) launch_pdl(rmsnorm_fwd_row_kernel<1>, dim3(T), dim3(256), 0, STREAM(stream), xp, rp, wp, hp, yp, rstd, d, eps);
  else if (nv == 2) launch_pdl(rmsnorm_fwd_row_kernel<2>, dim3(T), dim3(256), 0, STREAM(stream), xp, rp, wp, hp, yp, rstd, d, eps);
  else if (nv <= 4) launch_pdl(rmsnorm_fwd_row_kernel<4>, dim3(T), dim3(256), 0, STREAM(stream), xp, rp, wp, hp, yp, rstd, d, eps);
  else
    rmsnorm_fwd_kernel<<<(T + ROW_WARPS - 1) / ROW_WARPS, ROW_WARPS * 32, 0, STREAM(stream)>>>(xp, rp, wp, hp, yp, rstd, T, d, eps);
  return LAUNCH_OK();
}

extern "C" int rpeg_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd,
                                const void* dres_in, void* dx, float* dw, int T, int d, void* stream) {
  if (d & 7) return -2;
  if (T <= 0) return 0;
  const int nv = ((d >> 3) + 255) / 256;
  if (nv <= 2) {
    const __nv_bfloat16 *dyp = static_cast<const __nv_bfloat16*>(dy), *xp = static_cast<const __nv_bfloat16*>(x),
                        *wp = static_cast<const __nv_bfloat16*>(w), *rp = static_cast<const __nv_bfloat16*>(dres_in);
    __nv_bfloat16* dxp = static_cast<__nv_bfloat16*>(dx);
    const int grid = T < 1184 ? T : 1184;      // 8 resident CTAs on each of the 148 SMs
    if (nv == 1) rmsnorm_bwd_row_kernel<1><<<grid, 256, 0, STREAM(stream)>>>(dyp, xp, wp, rstd, rp, dxp, dw, T, d);
    else rmsnorm_bwd_row_kernel<2><<<grid, 256, 0, STREAM(stream)>>>(dyp, xp, wp, rstd, rp, dxp, dw, T, d);
    return LAUNCH_OK();
  }
  if (d * 4 > 200 * 1024) return -3;
  const int rows_per_cta = 32;
  auto kern = rmsnorm_bwd_kernel;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    configured = true;
  }
  kern<<<(T + rows_per_cta - 1) / rows_per_cta, ROW_WARPS * 32, d * 4, STREAM(stream)>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),
      static_cast<const __nv_bfloat16*>(w), rstd, static_cast<const __nv_bfloat16*>(dres_in),
      static_cast<__nv_bfloat16*>(dx), dw, T, d, rows_per_cta);
  return LAUNCH_OK();
}

extern "C" int rpeg_headnorm_fwd(void* buf, int ld, int col0, int nheads, int hd, const void* w, float* rstd, int T,
                                 float eps, void* stream) {
  if (hd != 128 || (ld & 3) || (col0 & 3)) return -2;
  const long long rows = static_cast<long long>(T) * nheads;
  if (rows <= 0) return 0;
  headnorm_fwd_kernel<<<static_cast<unsigned>((rows * 32 + 255) / 256), 256, 0, STREAM(stream)>>>(
      static_cast<__nv_bfloat16*>(buf), ld, col0, nheads, static_cast<const __nv_bfloat16*>(w), rstd, rows, eps);
  return LAUNCH_OK();
}

extern "C" int rpeg_headnorm_bwd(void* dbuf, int ldd, const void* x, int ldx, int col0, int nheads, int hd, const void* w,
                                 const float* rstd, float* dw, int T, void* stream) {
  if (hd != 128 || ((ldd | ldx | col0) & 3)) return -2;
  const long long rows = static_cast<long long>(T) * nheads;
  if (rows <= 0) return 0;
  long long blocks = (rows * 32 + 255) / 256;
  if (blocks > 1184) blocks = 1184;
  headnorm_bwd_kernel<<<static_cast<unsigned>(blocks), 256, 0, STREAM(stream)>>>(
      static_cast<__nv_bfloat16*>(dbuf), ldd, static_cast<const __nv_bfloat16*>(x), ldx, col0, nheads,
      static_cast<const __nv_bfloat16*>(w), rstd, dw, rows);
  return LAUNCH_OK();
}

extern "C" int rpeg_rmsnorm_fwd_partials(const float* parts, int splits, long long stride, const void* res, const void* w,
                                         void* h_out, void* y, int T, int d, float eps, void* stream) {
  if ((d & 7) || splits < 1) return -2;
  if (T <= 0) return 0;
  const __nv_bfloat16 *rp = static_cast<const __nv_bfloat16*>(res), *wp = static_cast<const __nv_bfloat16*>(w);
  __nv_bfloat16 *hp = static_cast<__nv_bfloat16*>(h_out), *yp = static_cast<__nv_bfloat16*>(y);
  const int nv = ((d >> 3) + 255) / 256;
  if (nv == 1) launch_pdl(rmsnorm_fwd_partials_kernel<1>, dim3(T), dim3(256), 0, STREAM(stream), parts, splits, stride, rp, wp, hp, yp, d, eps);
  else if (nv == 2) launch_pdl(rmsnorm_fwd_partials_kernel<2>, dim3(T), dim3(256), 0, STREAM(stream), parts, splits, stride, rp, wp, hp, yp, d, eps);
  else if (nv <= 4) launch_pdl(rmsnorm_fwd_partials_kernel<4>, dim3(T), dim3(256), 0, STREAM(stream), parts, splits, stride, rp, wp, hp, yp, d, eps);
  else return -3;
  return LAUNCH_OK();
}

extern "C" int rpeg_swiglu_fwd_partials(const float* parts, int splits, long long stride, void* out, long long T, int f,
                                        void* stream) {
  if ((f & 7) || splits < 1) return -2;
  const long long n = T * (f >> 3);
  if (n <= 0) return 0;
  launch_pdl(swiglu_fwd_partials_kernel, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0, STREAM(stream), 
      parts, splits, stride, static_cast<__nv_bfloat16*>(out), T, f);
  return LAUNCH_OK();
}

extern "C" int rpeg_rope(void* buf, const int* pos, const float* cos_t, const float* sin_t, int T, int ld,
                         int col0, int nheads, int hd, int backward, void* stream) {
  if ((hd & 3) || (ld & 1) || (col0 & 1)) return -2;
  const long long n = static_cast<long long>(T) * nheads * (hd >> 2);
  if (n <= 0) return 0;
  rope_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, STREAM(stream)>>>(
      static_cast<__nv_bfloat16*>(buf), pos, cos_t, sin_t, T, ld, col0, nheads, hd, backward ? -1.f : 1.f);
  return LAUNCH_OK();
}

extern "C" int rpeg_swiglu_fwd(const void* gu, void* out, long long T, int f, void* stream) {
  if (f & 7) return -2;
  const long long n = T * (f >> 3);
  if (n <= 0) return 0;
  swiglu_fwd_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, STREAM(stream)>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<__nv_bfloat16*>(out), T, f);
  return LAUNCH_OK();
}

extern "C" int rpeg_swiglu_bwd(const void* gu, const void* dout, void* dgu, long long T, int f, void* stream) {
  if (f & 7) return -2;
  const long long n = T * (f >> 3);
  if (n <= 0) return 0;
  swiglu_bwd_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, STREAM(stream)>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<const __nv_bfloat16*>(dout),
      static_cast<__nv_bfloat16*>(dgu), T, f);
  return LAUNCH_OK();
}

extern "C" int rpeg_add_bf16(const void* a, const void* b, void* out, long long n, void* stream) {
  if (n & 7) return -2;
  const long long nvec = n >> 3;
  if (nvec <= 0) return 0;
  add_bf16_kernel<<<static_cast<unsigned>((nvec + 255) / 256), 256, 0, STREAM(stream)>>>(
      static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b),
      static_cast<__nv_bfloat16*>(out), nvec);
  return LAUNCH_OK();
}

extern "C" int rpeg_embed_fwd(const int* ids, const void* table, void* out, int T, int d, void* stream) {
  if (d & 7) return -2;
  const long long n = static_cast<long long>(T) * (d >> 3);
  if (n <= 0) return 0;
  launch_pdl(embed_fwd_kernel, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0, STREAM(stream), 
      ids, static_cast<const __nv_bfloat16*>(table), static_cast<__nv_bfloat16*>(out), T, d);
  return LAUNCH_OK();
}

extern "C" int rpeg_embed_bwd(const int* ids, const void* dout, float* dtable, int T, int d, void* stream) {
  if (d & 1) return -2;
  const long long n = static_cast<long long>(T) * (d >> 1);
  if (n <= 0) return 0;
  embed_bwd_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, STREAM(stream)>>>(
      ids, static_cast<const __nv_bfloat16*>(dout), dtable, T, d);
  return LAUNCH_OK();
}
