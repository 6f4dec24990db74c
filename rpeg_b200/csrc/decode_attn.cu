// Paged KV cache append and paged decode attention (split-KV + combine) for sm_100a.
//
// Cache layout per layer: K pages and V pages, each [num_pages, H_kv, PAGE, hd] bf16 with PAGE = 64,
// so one (page, head) block is a contiguous 16 KiB: every key row read is a full 256-byte line.
// A page table [B, max_pages] maps (sequence, position / PAGE) to a page; finished sequences give
// their pages back to the allocator, so no compaction copy is ever needed.
//
// Decode attention is bandwidth bound (one query row per head): each CTA owns (head, sequence,
// split), its 4 warps stride over 32-key blocks with one key per lane for QK^T and 4 output
// columns per lane for PV, keeping an online-softmax state per warp that is merged in shared memory.
// With nsplit > 1 the partial (m, l, o) of every split goes to a scratch buffer and a second
// kernel merges them.
//
// Replaces the reference's static-KV decode: Megatron StaticInferenceContext plus per-layer
// index_select/copy compaction (RPEG/runtime/workers/megatron_worker.py:2585-2598, 2667-2811).
#include "common.cuh"
#include "rpeg_kernels.h"

namespace rpeg {

constexpr int PAGE = RPEG_KV_PAGE;
constexpr int HD = 128;

// Scatter new K/V rows of a packed [T, ld] qkv buffer into the paged cache.
//   token t belongs to sequence seq_id[t] at position pos[t].
__global__ void kv_append_kernel(const __nv_bfloat16* __restrict__ qkv, int ld, int k_col0, int v_col0,
                                 const int* __restrict__ seq_id, const int* __restrict__ pos,
                                 const int* __restrict__ page_table, int max_pages,
                                 __nv_bfloat16* __restrict__ kcache, __nv_bfloat16* __restrict__ vcache,
                                 int T, int Hkv) {
  // one thread per 16 bytes: T * Hkv * 16 vectors for K and the same for V
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long per_tok = static_cast<long long>(Hkv) * 16;
  if (idx >= static_cast<long long>(T) * per_tok) return;
  const int t = static_cast<int>(idx / per_tok);
  const int r = static_cast<int>(idx % per_tok);
  const int h = r >> 4, j = r & 15;
  const int p = pos[t];
  const int page = page_table[static_cast<size_t>(seq_id[t]) * max_pages + p / PAGE];
  const size_t dst = ((static_cast<size_t>(page) * Hkv + h) * PAGE + (p % PAGE)) * HD;
  const __nv_bfloat16* row = qkv + static_cast<size_t>(t) * ld;
  reinterpret_cast<uint4*>(kcache + dst)[j] = reinterpret_cast<const uint4*>(row + k_col0 + h * HD)[j];
  reinterpret_cast<uint4*>(vcache + dst)[j] = reinterpret_cast<const uint4*>(row + v_col0 + h * HD)[j];
}

struct WarpState {
  float m, l;
  float acc[4];
};

// q: [B, ldq] with head h at column q_col0 + h*HD. out: [B, H*HD] bf16.
// partial (when nsplit > 1): [B, H, nsplit, HD + 2] fp32 = {o[HD], m, l}.
__global__ void __launch_bounds__(128)
paged_decode_attn_kernel(const __nv_bfloat16* __restrict__ q, int ldq, int q_col0,
                         const __nv_bfloat16* __restrict__ kcache, const __nv_bfloat16* __restrict__ vcache,
                         const int* __restrict__ page_table, int max_pages, const int* __restrict__ seq_lens,
                         __nv_bfloat16* __restrict__ out, float* __restrict__ partial, int H, int Hkv,
                         int nsplit, float scale_log2) {
  __shared__ __align__(16) float q_sm[HD];
  __shared__ float red_m[4], red_l[4];
  __shared__ __align__(16) float red_o[4][HD];
  const int h = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
  const int hk = h / (H / Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int L = seq_lens[b];
  // split boundaries in units of 32-key blocks
  const int nblk = (L + 31) / 32;
  const int blk_per_split = (nblk + nsplit - 1) / nsplit;
  const int blk0 = split * blk_per_split;
  const int blk1 = min(nblk, blk0 + blk_per_split);

  if (threadIdx.x < HD)
    q_sm[threadIdx.x] = __bfloat162float(q[static_cast<size_t>(b) * ldq + q_col0 + h * HD + threadIdx.x]) * scale_log2;
  __syncthreads();

  float m = -INFINITY, l = 0.f;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  const int* pt = page_table + static_cast<size_t>(b) * max_pages;
  for (int blk = blk0 + warp; blk < blk1; blk += 4) {
    const int key = blk * 32 + lane;
    const int page = pt[(blk * 32) / PAGE];
    const size_t base = ((static_cast<size_t>(page) * Hkv + hk) * PAGE + ((blk * 32) % PAGE)) * HD;
    float s = -INFINITY;
    if (key < L) {
      const uint4* kr = reinterpret_cast<const uint4*>(kcache + base + static_cast<size_t>(lane) * HD);
      float d = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const uint4 kv = kr[i];
        const uint32_t* pk = reinterpret_cast<const uint32_t*>(&kv);
        const float4 q0 = *reinterpret_cast<const float4*>(&q_sm[i * 8]);
        const float4 q1 = *reinterpret_cast<const float4*>(&q_sm[i * 8 + 4]);
        const float2 a = unpack_bf16x2(pk[0]), bb = unpack_bf16x2(pk[1]), c = unpack_bf16x2(pk[2]),
                     e = unpack_bf16x2(pk[3]);
        d += a.x * q0.x + a.y * q0.y + bb.x * q0.z + bb.y * q0.w + c.x * q1.x + c.y * q1.y + e.x * q1.z + e.y * q1.w;
      }
      s = d;
    }
    const float bm = warp_max(s);
    const float nm = fmaxf(m, bm);
    const float alpha = exp2f(m - nm);  // m = -inf on the first block gives 0
    const float p = (key < L) ? exp2f(s - nm) : 0.f;
    l = l * alpha + warp_sum(p);
#pragma unroll
    for (int k = 0; k < 4; ++k) acc[k] *= alpha;
    m = nm;
    const int nk = min(32, L - blk * 32);
    const __nv_bfloat16* vb = vcache + base + lane * 4;
    for (int j = 0; j < nk; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const uint2 vv = *reinterpret_cast<const uint2*>(vb + static_cast<size_t>(j) * HD);
      const float2 v0 = unpack_bf16x2(vv.x), v1 = unpack_bf16x2(vv.y);
      acc[0] += pj * v0.x; acc[1] += pj * v0.y; acc[2] += pj * v1.x; acc[3] += pj * v1.y;
    }
  }
  // merge the 4 warps
  if (lane == 0) { red_m[warp] = m; red_l[warp] = l; }
  *reinterpret_cast<float4*>(&red_o[warp][lane * 4]) = make_float4(acc[0], acc[1], acc[2], acc[3]);
  __syncthreads();
  if (threadIdx.x < HD) {
    float gm = fmaxf(fmaxf(red_m[0], red_m[1]), fmaxf(red_m[2], red_m[3]));
    float gl = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float a = (red_m[w] == -INFINITY) ? 0.f : exp2f(red_m[w] - gm);
      gl += red_l[w] * a;
      o += red_o[w][threadIdx.x] * a;
    }
    if (nsplit == 1) {
      out[(static_cast<size_t>(b) * H + h) * HD + threadIdx.x] = __float2bfloat16(gl > 0.f ? o / gl : 0.f);
    } else {
      float* pp = partial + ((static_cast<size_t>(b) * H + h) * nsplit + split) * (HD + 2);
      pp[threadIdx.x] = o;
      if (threadIdx.x == 0) { pp[HD] = gm; pp[HD + 1] = gl; }
    }
  }
}

__global__ void __launch_bounds__(HD)
decode_combine_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out, int H, int nsplit) {
  const int h = blockIdx.x, b = blockIdx.y;
  const float* pp = partial + (static_cast<size_t>(b) * H + h) * nsplit * (HD + 2);
  float gm = -INFINITY;
  for (int s = 0; s < nsplit; ++s) gm = fmaxf(gm, pp[s * (HD + 2) + HD]);
  float gl = 0.f, o = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float ms = pp[s * (HD + 2) + HD];
    const float a = (ms == -INFINITY) ? 0.f : exp2f(ms - gm);
    gl += pp[s * (HD + 2) + HD + 1] * a;
    o += pp[s * (HD + 2) + threadIdx.x] * a;
  }
  out[(static_cast<size_t>(b) * H + h) * HD + threadIdx.x] = __float2bfloat16(gl > 0.f ? o / gl : 0.f);
}

}  // namespace rpeg

using namespace rpeg;
#define STREAM(s) reinterpret_cast<cudaStream_t>(s)
#define LAUNCH_OK() (cudaGetLastError() == cudaSuccess ? 0 : -21)

extern "C" int rpeg_kv_append(const void* qkv, int ld, int k_col0, int v_col0, const int* seq_id, const int* pos,
                              const int* page_table, int max_pages, void* kcache, void* vcache, int T, int Hkv,
                              int hd, void* stream) {
  if (hd != HD) return -2;
  if ((ld | k_col0 | v_col0) & 7) return -3;
  const long long n = static_cast<long long>(T) * Hkv * 16;
  if (n <= 0) return 0;
  kv_append_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, STREAM(stream)>>>(
      static_cast<const __nv_bfloat16*>(qkv), ld, k_col0, v_col0, seq_id, pos, page_table, max_pages,
      static_cast<__nv_bfloat16*>(kcache), static_cast<__nv_bfloat16*>(vcache), T, Hkv);
  return LAUNCH_OK();
}

extern "C" long long rpeg_decode_attn_scratch_bytes(int B, int H, int nsplit) {
  return nsplit <= 1 ? 0 : static_cast<long long>(B) * H * nsplit * (HD + 2) * 4;
}

extern "C" int rpeg_paged_decode_attn(const void* q, int ldq, int q_col0, const void* kcache, const void* vcache,
                                      const int* page_table, int max_pages, const int* seq_lens, void* out,
                                      float* scratch, int B, int H, int Hkv, int hd, int nsplit, float scale,
                                      void* stream) {
  if (hd != HD || H % Hkv != 0) return -2;
  if (nsplit < 1 || nsplit > 64) return -3;
  if (nsplit > 1 && scratch == nullptr) return -4;
  if (B <= 0) return 0;
  const float scale_log2 = scale * 1.4426950408889634f;
  paged_decode_attn_kernel<<<dim3(H, B, nsplit), 128, 0, STREAM(stream)>>>(
      static_cast<const __nv_bfloat16*>(q), ldq, q_col0, static_cast<const __nv_bfloat16*>(kcache),
      static_cast<const __nv_bfloat16*>(vcache), page_table, max_pages, seq_lens,
      static_cast<__nv_bfloat16*>(out), scratch, H, Hkv, nsplit, scale_log2);
  if (nsplit > 1)
    decode_combine_kernel<<<dim3(H, B), HD, 0, STREAM(stream)>>>(scratch, static_cast<__nv_bfloat16*>(out), H, nsplit);
  return LAUNCH_OK();
}
