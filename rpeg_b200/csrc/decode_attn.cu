// Paged KV cache append and paged decode attention (split-KV + combine) for sm_100a.
//
// Cache layout per layer: K pages and V pages, each [num_pages, H_kv, PAGE, hd] bf16 with PAGE = 64,
// so one (page, head) block is a contiguous 16 KiB: every key row read is a full 256-byte line.
// A page table [B, max_pages] maps (sequence, position / PAGE) to a page; finished sequences give
// their pages back to the allocator, so no compaction copy is ever needed.
//
// Decode attention is bandwidth bound (one query row per head): each CTA owns (head, sequence,
// split), its 4 warps stride over 32-key blocks, 16 lanes per key row so every load is a coalesced
// 256-byte line, keeping an online-softmax state per warp that is merged in shared memory.
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

// One launch for what decode does to a fresh qkv row: rotate the query heads in place, rotate the
// key heads (in place and into the cache) and copy the value heads into the cache. One warp per
// (token, head) job; jobs [0, H) are query heads, [H, H+Hkv) key heads, [H+Hkv, H+2Hkv) value heads.
// Rotate-half pairing: lane i rotates pairs (2i, 2i+1) with their partners at +hd/2 (hd = 128).
__global__ void __launch_bounds__(256)
rope_kv_append_kernel(__nv_bfloat16* __restrict__ qkv, int ld, int q_col0, int k_col0, int v_col0,
                      const int* __restrict__ seq_id, const int* __restrict__ pos,
                      const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                      const int* __restrict__ page_table, int max_pages, __nv_bfloat16* __restrict__ kcache,
                      __nv_bfloat16* __restrict__ vcache, int T, int H, int Hkv) {
  const int jobs = H + 2 * Hkv;
  const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (wid >= static_cast<long long>(T) * jobs) return;
  const int lane = threadIdx.x & 31;
  const int t = static_cast<int>(wid / jobs), job = static_cast<int>(wid % jobs);
  const int p = pos[t];
  __nv_bfloat16* row = qkv + static_cast<size_t>(t) * ld;
  size_t dst = 0;
  if (job >= H) {
    const int page = page_table[static_cast<size_t>(seq_id[t]) * max_pages + p / PAGE];
    const int hk = (job - H) % Hkv;
    dst = ((static_cast<size_t>(page) * Hkv + hk) * PAGE + (p % PAGE)) * HD;
  }
  if (job >= H + Hkv) {                      // value head: plain copy
    if (lane < 16)
      reinterpret_cast<uint4*>(vcache + dst)[lane] = reinterpret_cast<const uint4*>(row + v_col0 + (job - H - Hkv) * HD)[lane];
    return;
  }
  __nv_bfloat16* base = row + (job < H ? q_col0 + job * HD : k_col0 + (job - H) * HD);
  constexpr int half = HD / 2;
  const int i = lane * 2;
  const float2 c = *reinterpret_cast<const float2*>(cos_t + static_cast<size_t>(p) * half + i);
  const float2 s = *reinterpret_cast<const float2*>(sin_t + static_cast<size_t>(p) * half + i);
  const float2 a = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(base + i));
  const float2 b = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(base + i + half));
  const uint32_t lo = pack_bf16x2(a.x * c.x - b.x * s.x, a.y * c.y - b.y * s.y);
  const uint32_t hi = pack_bf16x2(b.x * c.x + a.x * s.x, b.y * c.y + a.y * s.y);
  *reinterpret_cast<uint32_t*>(base + i) = lo;
  *reinterpret_cast<uint32_t*>(base + i + half) = hi;
  if (job >= H) {
    *reinterpret_cast<uint32_t*>(kcache + dst + i) = lo;
    *reinterpret_cast<uint32_t*>(kcache + dst + i + half) = hi;
  }
}

// The same job list as rope_kv_append_kernel, but the qkv row is the sum of split-K partials
// (fp32 [splits][T][ld]): the head slice is summed, rounded to bf16, rotated (q, k) and stored: q into
// the bf16 qkv buffer the attention kernel reads, k and v into the paged cache.
__global__ void __launch_bounds__(256)
rope_kv_append_partials_kernel(const float* __restrict__ parts, int splits, long long stride, __nv_bfloat16* __restrict__ qkv,
                               int ld, int q_col0, int k_col0, int v_col0, const int* __restrict__ seq_id,
                               const int* __restrict__ pos, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                               const int* __restrict__ page_table, int max_pages, __nv_bfloat16* __restrict__ kcache,
                               __nv_bfloat16* __restrict__ vcache, int T, int H, int Hkv) {
  griddep_launch();
  griddep_wait();   // may have been scheduled under the previous kernel's tail: nothing is read or written before this
  const int jobs = H + 2 * Hkv;
  const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (wid >= static_cast<long long>(T) * jobs) return;
  const int lane = threadIdx.x & 31;
  const int t = static_cast<int>(wid / jobs), job = static_cast<int>(wid % jobs);
  const int p = pos[t];
  const int col = job < H ? q_col0 + job * HD : (job < H + Hkv ? k_col0 + (job - H) * HD : v_col0 + (job - H - Hkv) * HD);
  size_t dst = 0;
  if (job >= H) {
    const int page = page_table[static_cast<size_t>(seq_id[t]) * max_pages + p / PAGE];
    const int hk = (job - H) % Hkv;
    dst = ((static_cast<size_t>(page) * Hkv + hk) * PAGE + (p % PAGE)) * HD;
  }
  constexpr int half = HD / 2;
  const int i = lane * 2;
  // lane owns elements (i, i+1) and their rotation partners (i+half, i+half+1)
  float lo0 = 0.f, lo1 = 0.f, hi0 = 0.f, hi1 = 0.f;
  const size_t off = static_cast<size_t>(t) * ld + col;
  for (int s = 0; s < splits; ++s) {
    const float2 a = *reinterpret_cast<const float2*>(parts + s * stride + off + i);
    const float2 b = *reinterpret_cast<const float2*>(parts + s * stride + off + i + half);
    lo0 += a.x; lo1 += a.y; hi0 += b.x; hi1 += b.y;
  }
  uint32_t lo = pack_bf16x2(lo0, lo1), hi = pack_bf16x2(hi0, hi1);
  if (job < H + Hkv) {
    const float2 a = unpack_bf16x2(lo), b = unpack_bf16x2(hi);
    const float2 c = *reinterpret_cast<const float2*>(cos_t + static_cast<size_t>(p) * half + i);
    const float2 sn = *reinterpret_cast<const float2*>(sin_t + static_cast<size_t>(p) * half + i);
    lo = pack_bf16x2(a.x * c.x - b.x * sn.x, a.y * c.y - b.y * sn.y);
    hi = pack_bf16x2(b.x * c.x + a.x * sn.x, b.y * c.y + a.y * sn.y);
  }
  __nv_bfloat16* cache = job < H ? nullptr : (job < H + Hkv ? kcache : vcache);
  if (job < H) {
    __nv_bfloat16* base = qkv + off;
    *reinterpret_cast<uint32_t*>(base + i) = lo;
    *reinterpret_cast<uint32_t*>(base + i + half) = hi;
  } else {
    *reinterpret_cast<uint32_t*>(cache + dst + i) = lo;
    *reinterpret_cast<uint32_t*>(cache + dst + i + half) = hi;
  }
}

// 16 per-lane partial dot products (one per key of a half block) -> the full dot product of key
// `lane & 15` in every lane of a 16-lane group: at each level half of the values go to the partner.
__device__ __forceinline__ float transpose_reduce16(float (&v)[16], int lane) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const bool up = lane & 8;
    const float send = up ? v[i] : v[i + 8];
    const float keep = up ? v[i + 8] : v[i];
    v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const bool up = lane & 4;
    const float send = up ? v[i] : v[i + 4];
    const float keep = up ? v[i + 4] : v[i];
    v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const bool up = lane & 2;
    const float send = up ? v[i] : v[i + 2];
    const float keep = up ? v[i + 2] : v[i];
    v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
  }
  const bool up = lane & 1;
  const float send = up ? v[0] : v[1];
  const float keep = up ? v[1] : v[0];
  return keep + __shfl_xor_sync(0xffffffffu, send, 1);
}

__device__ __forceinline__ float dot8(const uint4& kv, const float (&q)[8]) {
  const float2 a = unpack_bf16x2(kv.x), b = unpack_bf16x2(kv.y), c = unpack_bf16x2(kv.z), d = unpack_bf16x2(kv.w);
  return a.x * q[0] + a.y * q[1] + b.x * q[2] + b.y * q[3] + c.x * q[4] + c.y * q[5] + d.x * q[6] + d.y * q[7];
}

__device__ __forceinline__ void axpy8(float (&acc)[8], float p, const uint4& vv) {
  const float2 a = unpack_bf16x2(vv.x), b = unpack_bf16x2(vv.y), c = unpack_bf16x2(vv.z), d = unpack_bf16x2(vv.w);
  acc[0] += p * a.x; acc[1] += p * a.y; acc[2] += p * b.x; acc[3] += p * b.y;
  acc[4] += p * c.x; acc[5] += p * c.y; acc[6] += p * d.x; acc[7] += p * d.y;
}

// q: [B, ldq] with head h at column q_col0 + h*HD. out: [B, H*HD] bf16.
// partial (when nsplit > 1): [B, H, nsplit, HD + 2] fp32 = {o[HD], m, l}.
//
// Work split inside a warp: the 32 lanes form two groups of 16; a group reads one 256-byte K (or
// V) row per load instruction, lane c of the group owning the 16-byte chunk c (head dims 8c..8c+7),
// so every global load is fully coalesced and a lane keeps 8 independent 16-byte loads in flight.
// Group g takes keys g*16..g*16+15 of a 32-key block; the 16 partial dot products of a lane are
// summed across the group by a transposing butterfly that leaves the score of key `lane` in lane
// `lane`, which is the layout the online softmax wants. For PV each lane accumulates its 8 head
// dims over the group's keys; the two groups are added at the end.
__global__ void __launch_bounds__(128)
paged_decode_attn_kernel(const __nv_bfloat16* __restrict__ q, int ldq, int q_col0,
                         const __nv_bfloat16* __restrict__ kcache, const __nv_bfloat16* __restrict__ vcache,
                         const int* __restrict__ page_table, int max_pages, const int* __restrict__ seq_lens,
                         __nv_bfloat16* __restrict__ out, float* __restrict__ partial, int H, int Hkv,
                         int nsplit, float scale_log2, const int* __restrict__ row_key0, int slot_base, int nslots,
                         int* __restrict__ arrive) {
  griddep_launch();
  griddep_wait();   // may have been scheduled under the previous kernel's tail: nothing is read or written before this
  __shared__ float red_m[4], red_l[4];
  __shared__ int is_last;
  __shared__ __align__(16) float red_o[4][HD];
  const int h = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
  const int hk = h / (H / Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = lane >> 4, c = lane & 15;
  const int L = seq_lens[b];
  const int nblk = (L + 31) / 32;                  // 32-key blocks
  // keys before row_key0[b] (a multiple of 64: whole shared prompt pages) are covered by the group kernel below,
  // which leaves its result in partial slot 0; this kernel then fills slots slot_base .. slot_base + nsplit - 1
  const int key0 = row_key0 != nullptr ? min(row_key0[b], L) : 0;
  const int blk_first = key0 / 32;
  const int blk_per_split = (max(nblk - blk_first, 0) + nsplit - 1) / nsplit;
  const int blk0 = blk_first + split * blk_per_split;
  const int blk1 = min(nblk, blk0 + blk_per_split);

  float qr[8];
  {
    const uint4 qv = *reinterpret_cast<const uint4*>(q + static_cast<size_t>(b) * ldq + q_col0 + h * HD + c * 8);
    const float2 a = unpack_bf16x2(qv.x), bb = unpack_bf16x2(qv.y), cc = unpack_bf16x2(qv.z), d = unpack_bf16x2(qv.w);
    qr[0] = a.x * scale_log2; qr[1] = a.y * scale_log2; qr[2] = bb.x * scale_log2; qr[3] = bb.y * scale_log2;
    qr[4] = cc.x * scale_log2; qr[5] = cc.y * scale_log2; qr[6] = d.x * scale_log2; qr[7] = d.y * scale_log2;
  }

  float m = -INFINITY, l = 0.f;
  float acc[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] = 0.f;
  const int* pt = page_table + static_cast<size_t>(b) * max_pages;
  for (int blk = blk0 + warp; blk < blk1; blk += 4) {
    const int page = pt[(blk * 32) / PAGE];
    // first row of this group's 16 keys, this lane's 16-byte chunk
    const size_t base = ((static_cast<size_t>(page) * Hkv + hk) * PAGE + ((blk * 32) % PAGE) + grp * 16) * HD + c * 8;
    const int nk = min(32, L - blk * 32) - grp * 16;   // valid keys of this group (may be <= 0)
    const uint4* kp = reinterpret_cast<const uint4*>(kcache + base);
    const uint4* vp = reinterpret_cast<const uint4*>(vcache + base);
    float part[16];
    if (nk >= 16) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint4 kv[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) kv[j] = kp[(half * 8 + j) * (HD / 8)];
#pragma unroll
        for (int j = 0; j < 8; ++j) part[half * 8 + j] = dot8(kv[j], qr);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        part[j] = 0.f;
        if (j < nk) part[j] = dot8(kp[j * (HD / 8)], qr);
      }
    }
    float s = transpose_reduce16(part, lane);       // score of key (blk*32 + lane)
    if (c >= nk) s = -INFINITY;
    const float bm = warp_max(s);
    const float nm = fmaxf(m, bm);
    const float alpha = exp2f(m - nm);              // m = -inf on the first block gives 0
    const float p = (c < nk) ? exp2f(s - nm) : 0.f;
    l = l * alpha + warp_sum(p);
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] *= alpha;
    m = nm;
    if (nk >= 16) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint4 vv[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) vv[j] = vp[(half * 8 + j) * (HD / 8)];
#pragma unroll
        for (int j = 0; j < 8; ++j) axpy8(acc, __shfl_sync(0xffffffffu, p, grp * 16 + half * 8 + j), vv[j]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float pj = __shfl_sync(0xffffffffu, p, grp * 16 + j);
        if (j < nk) axpy8(acc, pj, vp[j * (HD / 8)]);
      }
    }
  }
  // add the two key groups, then merge the 4 warps
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], 16);
  if (lane == 0) { red_m[warp] = m; red_l[warp] = l; }
  if (grp == 0) {
    *reinterpret_cast<float4*>(&red_o[warp][c * 8]) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4*>(&red_o[warp][c * 8 + 4]) = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
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
    if (nslots == 1) {
      out[(static_cast<size_t>(b) * H + h) * HD + threadIdx.x] = __float2bfloat16(gl > 0.f ? o / gl : 0.f);
    } else {
      float* pp = partial + ((static_cast<size_t>(b) * H + h) * nslots + slot_base + split) * (HD + 2);
      pp[threadIdx.x] = o;
      if (threadIdx.x == 0) { pp[HD] = gm; pp[HD + 1] = gl; }
      if (slot_base > 0 && split == 0 && key0 == 0) {       // no shared part for this row: slot 0 is empty
        float* p0 = partial + (static_cast<size_t>(b) * H + h) * nslots * (HD + 2);
        p0[threadIdx.x] = 0.f;
        if (threadIdx.x == 0) { p0[HD] = -INFINITY; p0[HD + 1] = 0.f; }
      }
    }
  }
  // Combine without a second kernel: the splits of a (row, head) count their arrivals; the last one merges all
  // partials (they are in L2 by then) and puts the counter back to zero for the next launch.
  if (arrive != nullptr && nslots > 1) {
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) is_last = (atomicAdd(&arrive[b * H + h], 1) == nsplit - 1) ? 1 : 0;
    __syncthreads();
    if (is_last) {
      if (threadIdx.x == 0) arrive[b * H + h] = 0;
      __threadfence();
      const float* pp = partial + (static_cast<size_t>(b) * H + h) * nslots * (HD + 2);
      float gm = -INFINITY;
      for (int s = 0; s < nslots; ++s) gm = fmaxf(gm, __ldcg(pp + s * (HD + 2) + HD));
      float gl = 0.f, o = 0.f;
      for (int s = 0; s < nslots; ++s) {
        const float ms = __ldcg(pp + s * (HD + 2) + HD);
        const float a = (ms == -INFINITY) ? 0.f : exp2f(ms - gm);
        gl += __ldcg(pp + s * (HD + 2) + HD + 1) * a;
        o += __ldcg(pp + s * (HD + 2) + threadIdx.x) * a;
      }
      out[(static_cast<size_t>(b) * H + h) * HD + threadIdx.x] = __float2bfloat16(gl > 0.f ? o / gl : 0.f);
    }
  }
}

// Arrival counters of the fused combine, one per (row, head); zero between launches. One split-KV decode attention
// launch at a time per GPU may use them (the kernels of a decode step run in stream order); larger batches and
// RPEG_DECODE_FUSED_COMBINE=0 use the separate combine kernel.
constexpr int ARRIVE_SLOTS = 1 << 16;
__device__ int g_decode_arrive[ARRIVE_SLOTS];

static int* fused_combine_counters(int B, int H) {
  static int on = -1;
  static int* ptr = nullptr;
  if (on < 0) {
    const char* e = getenv("RPEG_DECODE_FUSED_COMBINE");
    on = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  if (!on || static_cast<long long>(B) * H > ARRIVE_SLOTS) return nullptr;
  if (ptr == nullptr && cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_decode_arrive) != cudaSuccess) return nullptr;
  return ptr;
}

// Shared prompt pages: the K samples of one prompt alias the prompt's KV pages, so their queries can be scored
// against each K/V tile while it is in registers instead of streaming it once per row. One CTA per (head, group):
// group_rows[g][0..7] are the batch rows of the group (-1 = none, rows[0] is valid whenever group_shared[g] > 0),
// group_shared[g] the number of shared keys (a multiple of 64). Same lane layout as the per-row kernel; the 8
// queries sit in shared memory, their softmax state and output accumulators in registers. The result of every
// member row goes to partial slot 0 in the split-KV format {o[HD], m, l}; the per-row kernel covers the rest.
constexpr int GROUP_MAX = 8;

__global__ void __launch_bounds__(128)
paged_decode_attn_shared_kernel(const __nv_bfloat16* __restrict__ q, int ldq, int q_col0,
                                const __nv_bfloat16* __restrict__ kcache, const __nv_bfloat16* __restrict__ vcache,
                                const int* __restrict__ page_table, int max_pages, const int* __restrict__ group_rows,
                                const int* __restrict__ group_shared, float* __restrict__ partial, int H, int Hkv,
                                int nslots, float scale_log2) {
  griddep_launch();
  griddep_wait();   // may have been scheduled under the previous kernel's tail: nothing is read or written before this
  __shared__ __align__(16) float q_s[GROUP_MAX][HD];
  __shared__ float p_s[4][GROUP_MAX][32];
  __shared__ float red_m[4][GROUP_MAX], red_l[4][GROUP_MAX];
  __shared__ __align__(16) float red_o[4][GROUP_MAX][HD];
  __shared__ int rows_s[GROUP_MAX];
  const int h = blockIdx.x, g = blockIdx.y;
  const int S = group_shared[g];
  if (S <= 0) return;
  const int hk = h / (H / Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = lane >> 4, c = lane & 15;
  if (threadIdx.x < GROUP_MAX) rows_s[threadIdx.x] = group_rows[g * GROUP_MAX + threadIdx.x];
  __syncthreads();
#pragma unroll
  for (int qi = 0; qi < GROUP_MAX; ++qi) {
    const int r = rows_s[qi];
    q_s[qi][threadIdx.x] = r >= 0 ? __bfloat162float(q[static_cast<size_t>(r) * ldq + q_col0 + h * HD + threadIdx.x]) * scale_log2 : 0.f;
  }
  __syncthreads();
  const int leader = rows_s[0];
  const int* pt = page_table + static_cast<size_t>(leader) * max_pages;
  const int nblk = S / 32;

  float m[GROUP_MAX], l[GROUP_MAX], acc[GROUP_MAX][8];
#pragma unroll
  for (int qi = 0; qi < GROUP_MAX; ++qi) {
    m[qi] = -INFINITY;
    l[qi] = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[qi][k] = 0.f;
  }
  for (int blk = warp; blk < nblk; blk += 4) {
    const int page = pt[(blk * 32) / PAGE];
    const size_t base = ((static_cast<size_t>(page) * Hkv + hk) * PAGE + ((blk * 32) % PAGE) + grp * 16) * HD + c * 8;
    const uint4* kp = reinterpret_cast<const uint4*>(kcache + base);
    const uint4* vp = reinterpret_cast<const uint4*>(vcache + base);
    {
      uint4 kv[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) kv[j] = kp[j * (HD / 8)];
#pragma unroll
      for (int qi = 0; qi < GROUP_MAX; ++qi) {
        float qr[8];
        const float4 q0 = *reinterpret_cast<const float4*>(&q_s[qi][c * 8]);
        const float4 q1 = *reinterpret_cast<const float4*>(&q_s[qi][c * 8 + 4]);
        qr[0] = q0.x; qr[1] = q0.y; qr[2] = q0.z; qr[3] = q0.w; qr[4] = q1.x; qr[5] = q1.y; qr[6] = q1.z; qr[7] = q1.w;
        float part[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) part[j] = dot8(kv[j], qr);
        const float sc = transpose_reduce16(part, lane);     // score of key blk*32 + lane for query qi
        const float nm = fmaxf(m[qi], warp_max(sc));
        const float alpha = exp2f(m[qi] - nm);
        const float pr = exp2f(sc - nm);
        l[qi] = l[qi] * alpha + warp_sum(pr);
        m[qi] = nm;
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[qi][k] *= alpha;
        p_s[warp][qi][lane] = pr;
      }
    }
    __syncwarp();
    {
      uint4 vv[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) vv[j] = vp[j * (HD / 8)];
#pragma unroll
      for (int qi = 0; qi < GROUP_MAX; ++qi) {
#pragma unroll
        for (int j = 0; j < 16; ++j) axpy8(acc[qi], p_s[warp][qi][grp * 16 + j], vv[j]);
      }
    }
    __syncwarp();
  }
  // add the two key groups of a warp, then merge the 4 warps per query
#pragma unroll
  for (int qi = 0; qi < GROUP_MAX; ++qi) {
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[qi][k] += __shfl_xor_sync(0xffffffffu, acc[qi][k], 16);
    if (lane == 0) { red_m[warp][qi] = m[qi]; red_l[warp][qi] = l[qi]; }
    if (grp == 0) {
      *reinterpret_cast<float4*>(&red_o[warp][qi][c * 8]) = make_float4(acc[qi][0], acc[qi][1], acc[qi][2], acc[qi][3]);
      *reinterpret_cast<float4*>(&red_o[warp][qi][c * 8 + 4]) = make_float4(acc[qi][4], acc[qi][5], acc[qi][6], acc[qi][7]);
    }
  }
  __syncthreads();
  for (int qi = 0; qi < GROUP_MAX; ++qi) {
    const int r = rows_s[qi];
    if (r < 0) continue;
    const float gm = fmaxf(fmaxf(red_m[0][qi], red_m[1][qi]), fmaxf(red_m[2][qi], red_m[3][qi]));
    float gl = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float a = (red_m[w][qi] == -INFINITY) ? 0.f : exp2f(red_m[w][qi] - gm);
      gl += red_l[w][qi] * a;
      o += red_o[w][qi][threadIdx.x] * a;
    }
    float* pp = partial + (static_cast<size_t>(r) * H + h) * nslots * (HD + 2);
    pp[threadIdx.x] = o;
    if (threadIdx.x == 0) { pp[HD] = gm; pp[HD + 1] = gl; }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// The same job on the tensor cores. One persistent CTA per SM walks the (group, head) items; the shared keys of an item
// are streamed ONCE through a ring of {K tile, V tile} stages (TMA, 128 keys = two pages per tile) and scored against
// all queries of the group by tcgen05.mma with the KEYS on the M axis:
//     S^T [128 keys x 16]  = K tile [128 x 128 hd] (A, K-major)  x  Q^T (B: 16 query rows x 128 hd, rows 8..15 zero)
//     O^T [128 hd   x 16] += V^T    [128 hd x 128 keys] (A, MN-major: the V tile as stored)  x  P^T (B: 16 x 128 keys)
// Softmax threads own one key (= TMEM lane) each: the per-query maximum over a tile is a warp shuffle plus a four-way
// exchange through shared memory; the running maximum is refreshed lazily (only when it grows by more than 8 in log2
// units), so O is rarely rescaled. P goes to shared memory in the B-operand layout. S, P and O are double buffered
// (S and P by tile, O and Q by item), the next item's Q is staged while the current item runs, and the producer runs
// ahead across item boundaries, so the HBM stream never stops between items. Output format and the rest of the row
// (per-row kernel, combine) are those of the CUDA-core version above.
constexpr int GT_THREADS = 192;
constexpr int GT_STAGES = 3;
constexpr int GT_TILE = 128;                       // keys per tile
constexpr int GT_HALF_BYTES = 64 * 64 * 2;         // one TMA box: 64 rows x 64 columns bf16 = 8 KiB
constexpr int GT_KV_BYTES = 128 * HD * 2;          // 32 KiB: one K (or V) tile
constexpr int GT_STAGE_BYTES = 2 * GT_KV_BYTES;
constexpr int GT_QP_BYTES = 16 * HD * 2;           // 4 KiB: 16 rows x 128 elements, two 64-column atoms of 2 KiB
constexpr int GT_SMEM = GT_STAGES * GT_STAGE_BYTES + 4 * GT_QP_BYTES + 1024 /*align*/ + 1024 /*barriers, exchange*/;
constexpr float GT_RESCALE_THRESHOLD = 8.0f;

__device__ __forceinline__ void tmem_ld_32x8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_st_32x8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(r[0]),
               "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}

__global__ void __launch_bounds__(GT_THREADS, 1)
paged_decode_attn_shared_tc_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                                   const __nv_bfloat16* __restrict__ q, int ldq, int q_col0,
                                   const int* __restrict__ page_table, int max_pages, const int* __restrict__ group_rows,
                                   const int* __restrict__ group_shared, float* __restrict__ partial, int n_groups, int H,
                                   int Hkv, int nslots, float scale_log2, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ring = smem;
  uint8_t* q_sm = ring + GT_STAGES * GT_STAGE_BYTES;      // [2][4 KiB]
  uint8_t* p_sm = q_sm + 2 * GT_QP_BYTES;                 // [2][4 KiB]
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_sm + 2 * GT_QP_BYTES);
  uint64_t* kv_full = bars;                  // [3]
  uint64_t* kv_empty = kv_full + GT_STAGES;  // [3]
  uint64_t* s_full = kv_empty + GT_STAGES;   // [2] by tile parity
  uint64_t* p_full = s_full + 2;             // [2] by tile parity, 4 arrivals
  uint64_t* pv_done = p_full + 2;            // [2] by tile parity
  uint64_t* q_full = pv_done + 2;            // [2] by item parity, 4 arrivals
  uint64_t* o_free = q_full + 2;             // [2] by item parity, 4 arrivals
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_free + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* red = reinterpret_cast<float*>(tmem_slot + 4);   // [4 warps][8 queries]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < GT_STAGES; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&s_full[b], 1); mbar_init(&p_full[b], 4); mbar_init(&pv_done[b], 1);
      mbar_init(&q_full[b], 4); mbar_init(&o_free[b], 4);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  // Zero the operand buffers once: rows 8..15 of Q and P stay zero for good, and a tile whose second page does not
  // exist multiplies stale but finite V rows by probabilities of exactly zero.
  for (int i = threadIdx.x; i < (GT_STAGES * GT_STAGE_BYTES + 4 * GT_QP_BYTES) / 16; i += GT_THREADS)
    reinterpret_cast<uint4*>(ring)[i] = make_uint4(0u, 0u, 0u, 0u);
  fence_proxy_async_smem();
  if (warp == 1) {
    tmem_alloc(tmem_slot, 64);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  griddep_launch();
  griddep_wait();   // everything above touched only this CTA's own memory

  const int n_items = n_groups * H;
  const int G = H / Hkv;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmap_k);
      tma_prefetch_desc(&tmap_v);
      int t = 0;
      for (int w = blockIdx.x; w < n_items; w += gridDim.x) {
        const int g = w / H, h = w % H;
        const int S = group_shared[g];
        if (S <= 0) continue;
        const int hk = h / G;
        const int* pt = page_table + static_cast<size_t>(group_rows[g * GROUP_MAX]) * max_pages;
        const int n_pages = S / PAGE;
        for (int j = 0; j * 2 < n_pages; ++j, ++t) {
          const int st = t % GT_STAGES;
          const uint32_t ph = static_cast<uint32_t>(t / GT_STAGES) & 1u;
          if (!mbar_wait(&kv_empty[st], ph ^ 1u, abort_flag, status, 800)) goto producer_done;
          const int halves = (2 * j + 1 < n_pages) ? 2 : 1;
          mbar_expect_tx(&kv_full[st], static_cast<uint32_t>(halves * 4 * GT_HALF_BYTES));
          uint8_t* ks = ring + st * GT_STAGE_BYTES;
          uint8_t* vs = ks + GT_KV_BYTES;
          for (int hf = 0; hf < halves; ++hf) {
            const int row0 = (pt[2 * j + hf] * Hkv + hk) * PAGE;     // first row of the (page, head) block
            tma_load_2d(ks + hf * GT_HALF_BYTES, &tmap_k, &kv_full[st], 0, row0);
            tma_load_2d(ks + 16384 + hf * GT_HALF_BYTES, &tmap_k, &kv_full[st], 64, row0);
            tma_load_2d(vs + hf * GT_HALF_BYTES, &tmap_v, &kv_full[st], 0, row0);
            tma_load_2d(vs + 16384 + hf * GT_HALF_BYTES, &tmap_v, &kv_full[st], 64, row0);
          }
        }
      }
    producer_done:;
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t id_qk = make_idesc_bf16(128, 16, 0, 0);
      constexpr uint32_t id_pv = make_idesc_bf16(128, 16, 1, 0);   // A = V tile read MN-major
      // flat list of this CTA's tiles: (item number, tile in item, tiles of the item) are advanced together
      int w = blockIdx.x, it = -1, j = 0, nt = 0;
      auto next_tile = [&]() -> bool {     // moves (w, it, j, nt) to the next tile; false when the items are used up
        if (it >= 0 && j + 1 < nt) { ++j; return true; }
        if (it >= 0) w += gridDim.x;
        for (; w < n_items; w += gridDim.x) {
          const int S = group_shared[w / H];
          if (S > 0) { ++it; j = 0; nt = (S / PAGE + 1) / 2; return true; }
        }
        return false;
      };
      auto issue_qk = [&](int t, int item, int tile_j) -> bool {
        const int st = t % GT_STAGES;
        if (tile_j == 0 && !mbar_wait(&q_full[item & 1], static_cast<uint32_t>(item >> 1) & 1u, abort_flag, status, 810)) return false;
        if (!mbar_wait(&kv_full[st], static_cast<uint32_t>(t / GT_STAGES) & 1u, abort_flag, status, 811)) return false;
        tc_fence_after_sync();
        const uint32_t ka = smem_u32(ring + st * GT_STAGE_BYTES);
        const uint32_t qa = smem_u32(q_sm + (item & 1) * GT_QP_BYTES);
        const uint32_t ts = tmem_base + static_cast<uint32_t>((t & 1) * 16);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_bf16_ss(ts, make_smem_desc_sw128(ka + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024),
                       make_smem_desc_sw128(qa + (k >> 2) * 2048 + (k & 3) * 32, 16, 1024), id_qk, k != 0 ? 1u : 0u);
        umma_commit(&s_full[t & 1]);
        return true;
      };
      if (next_tile()) {
        int t = 0;
        bool ok = issue_qk(0, it, j);
        while (ok) {
          const int cur_it = it, cur_j = j;
          const bool more = next_tile();
          if (more && !issue_qk(t + 1, it, j)) break;                // S of the next tile is computed under this tile's softmax
          if (!mbar_wait(&p_full[t & 1], static_cast<uint32_t>(t >> 1) & 1u, abort_flag, status, 812)) break;
          if (cur_j == 0 && cur_it >= 2 &&
              !mbar_wait(&o_free[cur_it & 1], (static_cast<uint32_t>(cur_it >> 1) & 1u) ^ 1u, abort_flag, status, 813)) break;
          tc_fence_after_sync();
          const int st = t % GT_STAGES;
          const uint32_t va = smem_u32(ring + st * GT_STAGE_BYTES + GT_KV_BYTES);
          const uint32_t pa = smem_u32(p_sm + (t & 1) * GT_QP_BYTES);
          const uint32_t to = tmem_base + 32u + static_cast<uint32_t>((cur_it & 1) * 16);
#pragma unroll
          for (int k = 0; k < 8; ++k)      // 16 keys per step
            umma_bf16_ss(to, make_smem_desc_sw128(va + k * 2048, 16384, 1024),
                         make_smem_desc_sw128(pa + (k >> 2) * 2048 + (k & 3) * 32, 16, 1024), id_pv, (cur_j | k) != 0 ? 1u : 0u);
          umma_commit(&kv_empty[st]);
          umma_commit(&pv_done[t & 1]);
          if (!more) break;
          ++t;
        }
      }
    }
  } else {
    const int quad = warp & 3;
    const int r = quad * 32 + lane;                    // key inside a tile (softmax), head dim (O^T)
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const int tq = threadIdx.x - 64;                   // 0..127
    auto stage_q = [&](int item_w, int item_no) {      // 8 rows x 16 chunks of 16 bytes: one chunk per thread
      const int g = item_w / H, h = item_w % H;
      const int row = tq >> 4, chunk = tq & 15;
      const int br = group_rows[g * GROUP_MAX + row];
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (br >= 0) v = *reinterpret_cast<const uint4*>(q + static_cast<size_t>(br) * ldq + q_col0 + h * HD + chunk * 8);
      uint8_t* dst = q_sm + (item_no & 1) * GT_QP_BYTES + (chunk >> 3) * 2048 + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
      *reinterpret_cast<uint4*>(dst) = v;
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&q_full[item_no & 1]);
    };
    auto next_item = [&](int w0) -> int {              // first valid item at or after w0 in this CTA's sequence
      for (int w = w0; w < n_items; w += gridDim.x)
        if (group_shared[w / H] > 0) return w;
      return -1;
    };
    int w = next_item(blockIdx.x);
    if (w >= 0) stage_q(w, 0);
    int t = 0;
    bool ok = true;
    for (int it = 0; w >= 0 && ok; ++it) {
      const int w_next = next_item(w + gridDim.x);
      if (w_next >= 0) stage_q(w_next, it + 1);        // Q buffer (it+1)&1 was last read by item it-1, whose MMAs are complete
      const int g = w / H, h = w % H;
      const int S = group_shared[g];
      const int nt = (S / PAGE + 1) / 2;
      float m[GROUP_MAX], l[GROUP_MAX];
#pragma unroll
      for (int qi = 0; qi < GROUP_MAX; ++qi) { m[qi] = -INFINITY; l[qi] = 0.f; }
      const uint32_t t_o = tmem_base + 32u + static_cast<uint32_t>((it & 1) * 16) + lane_base;
      for (int j = 0; j < nt; ++j, ++t) {
        if (!__all_sync(0xffffffffu, mbar_wait(&s_full[t & 1], static_cast<uint32_t>(t >> 1) & 1u, abort_flag, status, 820))) { ok = false; break; }
        tc_fence_after_sync();
        uint32_t sv[8];
        tmem_ld_32x8(tmem_base + static_cast<uint32_t>((t & 1) * 16) + lane_base, sv);
        tmem_wait_ld();
        const bool key_valid = j * GT_TILE + r < S;
        float sc[GROUP_MAX];
#pragma unroll
        for (int qi = 0; qi < GROUP_MAX; ++qi) {
          sc[qi] = key_valid ? __uint_as_float(sv[qi]) * scale_log2 : -INFINITY;
          const float wm = warp_max(sc[qi]);
          if (lane == 0) red[quad * GROUP_MAX + qi] = wm;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        float tmax[GROUP_MAX];
        bool need = false;
#pragma unroll
        for (int qi = 0; qi < GROUP_MAX; ++qi) {
          tmax[qi] = fmaxf(fmaxf(red[qi], red[GROUP_MAX + qi]), fmaxf(red[2 * GROUP_MAX + qi], red[3 * GROUP_MAX + qi]));
          if (j == 0) m[qi] = tmax[qi];
          else need = need || (tmax[qi] > m[qi] + GT_RESCALE_THRESHOLD);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");     // `red` may be rewritten by the next tile
        if (need) {                                        // the same decision in every thread: all hold the same m and tmax
          // PV of the previous tile must have landed before O is rescaled. Having seen s_full of this tile, the waiter
          // is at most one completion behind on the barrier of that parity (see flash_attn_fwd_kernel).
          if (!__all_sync(0xffffffffu, mbar_wait(&pv_done[(t - 1) & 1], static_cast<uint32_t>((t - 1) >> 1) & 1u, abort_flag, status, 821))) { ok = false; break; }
          tc_fence_after_sync();
          float alpha[GROUP_MAX];
#pragma unroll
          for (int qi = 0; qi < GROUP_MAX; ++qi) {
            const float nm = fmaxf(m[qi], tmax[qi]);
            alpha[qi] = exp2f(m[qi] - nm);
            m[qi] = nm;
            l[qi] *= alpha[qi];
          }
          uint32_t ov[8];
          tmem_ld_32x8(t_o, ov);
          tmem_wait_ld();
#pragma unroll
          for (int qi = 0; qi < GROUP_MAX; ++qi) ov[qi] = __float_as_uint(__uint_as_float(ov[qi]) * alpha[qi]);
          tmem_st_32x8(t_o, ov);
          tmem_wait_st();
          tc_fence_before_sync();
        }
        // P^T in the B-operand layout: row = query, 128 keys contiguous (two 64-key atoms), 128-byte swizzle
        uint8_t* pb = p_sm + (t & 1) * GT_QP_BYTES + (r >> 6) * 2048 + (r & 7) * 2;
        const int chunk = (r & 63) >> 3;
#pragma unroll
        for (int qi = 0; qi < GROUP_MAX; ++qi) {
          const float pr = exp2f(sc[qi] - m[qi]);          // masked keys: exp2(-inf) = 0
          l[qi] += pr;
          *reinterpret_cast<__nv_bfloat16*>(pb + qi * 128 + ((chunk ^ qi) << 4)) = __float2bfloat16(pr);
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[t & 1]);
      }
      if (!ok) break;
      // item epilogue: this thread is head dim r of O^T; l is summed over the 128 key owners
      if (!__all_sync(0xffffffffu, mbar_wait(&pv_done[(t - 1) & 1], static_cast<uint32_t>((t - 1) >> 1) & 1u, abort_flag, status, 822))) { ok = false; break; }
      tc_fence_after_sync();
      uint32_t ov[8];
      tmem_ld_32x8(t_o, ov);
      tmem_wait_ld();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&o_free[it & 1]);
#pragma unroll
      for (int qi = 0; qi < GROUP_MAX; ++qi) {
        const float ws = warp_sum(l[qi]);
        if (lane == 0) red[quad * GROUP_MAX + qi] = ws;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
      for (int qi = 0; qi < GROUP_MAX; ++qi) {
        const int br = group_rows[g * GROUP_MAX + qi];
        if (br < 0) continue;
        float* pp = partial + (static_cast<size_t>(br) * H + h) * nslots * (HD + 2);
        pp[r] = __uint_as_float(ov[qi]);
        if (r == 0) {
          pp[HD] = m[qi];
          pp[HD + 1] = red[qi] + red[GROUP_MAX + qi] + red[2 * GROUP_MAX + qi] + red[3 * GROUP_MAX + qi];
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      w = w_next;
    }
  }

  __syncwarp();
  if (*abort_flag) __nanosleep(200000);
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 64);
  }
}

__global__ void __launch_bounds__(HD)
decode_combine_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out, int H, int nsplit) {
  griddep_launch();
  griddep_wait();   // may have been scheduled under the previous kernel's tail: nothing is read or written before this
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

extern "C" int rpeg_rope_kv_append(void* qkv, int ld, int q_col0, int k_col0, int v_col0, const int* seq_id, const int* pos,
                                   const float* cos_t, const float* sin_t, const int* page_table, int max_pages,
                                   void* kcache, void* vcache, int T, int H, int Hkv, int hd, void* stream) {
  if (hd != HD) return -2;
  if ((ld | q_col0 | k_col0 | v_col0) & 7) return -3;
  const long long threads = static_cast<long long>(T) * (H + 2 * Hkv) * 32;
  if (threads <= 0) return 0;
  rope_kv_append_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, STREAM(stream)>>>(
      static_cast<__nv_bfloat16*>(qkv), ld, q_col0, k_col0, v_col0, seq_id, pos, cos_t, sin_t, page_table, max_pages,
      static_cast<__nv_bfloat16*>(kcache), static_cast<__nv_bfloat16*>(vcache), T, H, Hkv);
  return LAUNCH_OK();
}

extern "C" int rpeg_rope_kv_append_partials(const float* parts, int splits, long long stride, void* qkv, int ld, int q_col0,
                                            int k_col0, int v_col0, const int* seq_id, const int* pos, const float* cos_t,
                                            const float* sin_t, const int* page_table, int max_pages, void* kcache,
                                            void* vcache, int T, int H, int Hkv, int hd, void* stream) {
  if (hd != HD || splits < 1) return -2;
  if ((ld | q_col0 | k_col0 | v_col0) & 7) return -3;
  const long long threads = static_cast<long long>(T) * (H + 2 * Hkv) * 32;
  if (threads <= 0) return 0;
  launch_pdl(rope_kv_append_partials_kernel, dim3(static_cast<unsigned>((threads + 255) / 256)), dim3(256), 0, STREAM(stream), 
      parts, splits, stride, static_cast<__nv_bfloat16*>(qkv), ld, q_col0, k_col0, v_col0, seq_id, pos, cos_t, sin_t, page_table,
      max_pages, static_cast<__nv_bfloat16*>(kcache), static_cast<__nv_bfloat16*>(vcache), T, H, Hkv);
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
  int* arrive = nsplit > 1 ? fused_combine_counters(B, H) : nullptr;
  launch_pdl(paged_decode_attn_kernel, dim3(dim3(H, B, nsplit)), dim3(128), 0, STREAM(stream), 
      static_cast<const __nv_bfloat16*>(q), ldq, q_col0, static_cast<const __nv_bfloat16*>(kcache),
      static_cast<const __nv_bfloat16*>(vcache), page_table, max_pages, seq_lens,
      static_cast<__nv_bfloat16*>(out), scratch, H, Hkv, nsplit, scale_log2, static_cast<const int*>(nullptr), 0, nsplit, arrive);
  if (nsplit > 1 && arrive == nullptr)
    launch_pdl(decode_combine_kernel, dim3(dim3(H, B)), dim3(HD), 0, STREAM(stream), scratch, static_cast<__nv_bfloat16*>(out), H, nsplit);
  return LAUNCH_OK();
}

// Decode attention for batches in which groups of rows share their first keys (K samples of one prompt aliasing
// the prompt's KV pages). group_rows [B, 8] (batch rows of group g, -1 padded; unused groups all -1), group_shared
// [B] (shared keys of group g, a multiple of 64, 0 = unused), row_key0 [B] (shared keys of ROW b, 0 if the row is in
// no group). The shared keys are read once per group, the rest once per row; the two parts meet in the split-KV
// combine. scratch: rpeg_decode_attn_scratch_bytes(B, H, nsplit + 1).
extern "C" int rpeg_paged_decode_attn_grouped(const void* q, int ldq, int q_col0, const void* kcache, const void* vcache,
                                              const int* page_table, int max_pages, const int* seq_lens, void* out,
                                              float* scratch, int B, int H, int Hkv, int hd, int nsplit, float scale,
                                              const int* group_rows, const int* group_shared, const int* row_key0,
                                              void* stream) {
  if (hd != HD || H % Hkv != 0) return -2;
  if (nsplit < 1 || nsplit > 63) return -3;
  if (scratch == nullptr || group_rows == nullptr || group_shared == nullptr || row_key0 == nullptr) return -4;
  if (B <= 0) return 0;
  const float scale_log2 = scale * 1.4426950408889634f;
  const int nslots = nsplit + 1;
  int* arrive = fused_combine_counters(B, H);
  launch_pdl(paged_decode_attn_shared_kernel, dim3(H, B), dim3(128), 0, STREAM(stream), static_cast<const __nv_bfloat16*>(q), ldq,
             q_col0, static_cast<const __nv_bfloat16*>(kcache), static_cast<const __nv_bfloat16*>(vcache), page_table, max_pages,
             group_rows, group_shared, scratch, H, Hkv, nslots, scale_log2);
  launch_pdl(paged_decode_attn_kernel, dim3(H, B, nsplit), dim3(128), 0, STREAM(stream), static_cast<const __nv_bfloat16*>(q), ldq,
             q_col0, static_cast<const __nv_bfloat16*>(kcache), static_cast<const __nv_bfloat16*>(vcache), page_table, max_pages,
             seq_lens, static_cast<__nv_bfloat16*>(out), scratch, H, Hkv, nsplit, scale_log2, row_key0, 1, nslots, arrive);
  if (arrive == nullptr)
    launch_pdl(decode_combine_kernel, dim3(H, B), dim3(HD), 0, STREAM(stream), scratch, static_cast<__nv_bfloat16*>(out), H, nslots);
  return LAUNCH_OK();
}

namespace rpeg {
int make_tmap_bf16_2d(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_inner,
                      uint32_t box_outer);
}

// rpeg_paged_decode_attn_grouped with the shared keys on the tensor cores (paged_decode_attn_shared_tc_kernel).
// `num_pages` is the page count of the K / V pools (bounds of the TMA descriptors).
extern "C" int rpeg_paged_decode_attn_grouped_tc(const void* q, int ldq, int q_col0, const void* kcache, const void* vcache,
                                                 long long num_pages, const int* page_table, int max_pages, const int* seq_lens,
                                                 void* out, float* scratch, int B, int H, int Hkv, int hd, int nsplit, float scale,
                                                 const int* group_rows, const int* group_shared, const int* row_key0, int* status,
                                                 void* stream) {
  if (hd != HD || H % Hkv != 0) return -2;
  if (nsplit < 1 || nsplit > 63) return -3;
  if (scratch == nullptr || group_rows == nullptr || group_shared == nullptr || row_key0 == nullptr) return -4;
  if ((ldq | q_col0) & 7) return -5;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(kcache) | reinterpret_cast<uintptr_t>(vcache)) & 15) return -1;
  if (B <= 0) return 0;
  const float scale_log2 = scale * 1.4426950408889634f;
  const int nslots = nsplit + 1;
  int* arrive = fused_combine_counters(B, H);
  CUtensorMap tk, tv;
  const uint64_t rows = static_cast<uint64_t>(num_pages) * Hkv * PAGE;
  int rc = make_tmap_bf16_2d(&tk, kcache, HD, rows, HD, 64, 64);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tv, vcache, HD, rows, HD, 64, 64);
  if (rc) return rc - 100;
  static bool configured = false;
  static int num_sms = 0;
  if (!configured) {
    if (cudaFuncSetAttribute(paged_decode_attn_shared_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GT_SMEM) != cudaSuccess)
      return -20;
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
    configured = true;
  }
  const int items = B * H;
  const int grid = items < num_sms ? items : num_sms;
  launch_pdl(paged_decode_attn_shared_tc_kernel, dim3(grid), dim3(GT_THREADS), GT_SMEM, STREAM(stream), tk, tv,
             static_cast<const __nv_bfloat16*>(q), ldq, q_col0, page_table, max_pages, group_rows, group_shared, scratch, B, H, Hkv,
             nslots, scale_log2, status);
  launch_pdl(paged_decode_attn_kernel, dim3(H, B, nsplit), dim3(128), 0, STREAM(stream), static_cast<const __nv_bfloat16*>(q), ldq,
             q_col0, static_cast<const __nv_bfloat16*>(kcache), static_cast<const __nv_bfloat16*>(vcache), page_table, max_pages,
             seq_lens, static_cast<__nv_bfloat16*>(out), scratch, H, Hkv, nsplit, scale_log2, row_key0, 1, nslots, arrive);
  if (arrive == nullptr)
    launch_pdl(decode_combine_kernel, dim3(H, B), dim3(HD), 0, STREAM(stream), scratch, static_cast<__nv_bfloat16*>(out), H, nslots);
  return LAUNCH_OK();
}

// ---------------------------------------------------------------------------------------------------
// Allocation-free variant: the split-KV partials live in a fixed device array of this library.
// Rules for callers are in decode_attn_static.h.
#include "decode_attn_static.h"

namespace {
constexpr long long STATIC_PARTIAL_FLOATS = static_cast<long long>(RPEG_DECODE_STATIC_MAX_PARTIALS) * (HD + 2);
static __device__ __align__(256) float g_decode_static_scratch[STATIC_PARTIAL_FLOATS];
constexpr int STATIC_MAX_DEVICES = 64;
float* g_static_scratch_ptr[STATIC_MAX_DEVICES] = {nullptr};
}  // namespace

extern "C" const char* rpeg_static_entry_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case RPEG_STATIC_ERR_BAD_SHAPE: return "unsupported shape: head_dim must be 128 and H a multiple of Hkv";
    case RPEG_STATIC_ERR_BAD_SPLIT: return "nsplit must be between 1 and 64";
    case RPEG_STATIC_ERR_TOO_LARGE:
      return "B * H * nsplit exceeds RPEG_DECODE_STATIC_MAX_PARTIALS (16384): the built-in scratch is too small for this call";
    case RPEG_STATIC_ERR_SETUP: return "set-up failed: the address of the built-in scratch could not be obtained on this device";
    case RPEG_STATIC_ERR_LAUNCH: return "kernel launch failed";
    default: return "unknown code";
  }
}

extern "C" int rpeg_paged_decode_attn_static(const void* q, int ldq, int q_col0, const void* kcache, const void* vcache,
                                             const int* page_table, int max_pages, const int* seq_lens, void* out,
                                             int B, int H, int Hkv, int hd, int nsplit, float scale, void* stream) {
  if (hd != HD || Hkv <= 0 || H % Hkv != 0) return RPEG_STATIC_ERR_BAD_SHAPE;
  if (nsplit < 1 || nsplit > 64) return RPEG_STATIC_ERR_BAD_SPLIT;
  if (B <= 0) return 0;
  if (static_cast<long long>(B) * H * nsplit > RPEG_DECODE_STATIC_MAX_PARTIALS) return RPEG_STATIC_ERR_TOO_LARGE;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= STATIC_MAX_DEVICES) return RPEG_STATIC_ERR_SETUP;
  if (g_static_scratch_ptr[dev] == nullptr) {
    // set-up, once per device: the array's address in this device's copy of the module
    float* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_decode_static_scratch) != cudaSuccess || p == nullptr)
      return RPEG_STATIC_ERR_SETUP;
    g_static_scratch_ptr[dev] = p;
  }
  float* scratch = g_static_scratch_ptr[dev];
  const float scale_log2 = scale * 1.4426950408889634f;
  launch_pdl(paged_decode_attn_kernel, dim3(dim3(H, B, nsplit)), dim3(128), 0, STREAM(stream), 
      static_cast<const __nv_bfloat16*>(q), ldq, q_col0, static_cast<const __nv_bfloat16*>(kcache),
      static_cast<const __nv_bfloat16*>(vcache), page_table, max_pages, seq_lens, static_cast<__nv_bfloat16*>(out),
      scratch, H, Hkv, nsplit, scale_log2, static_cast<const int*>(nullptr), 0, nsplit, static_cast<int*>(nullptr));
  if (nsplit > 1)
    launch_pdl(decode_combine_kernel, dim3(dim3(H, B)), dim3(HD), 0, STREAM(stream), scratch, static_cast<__nv_bfloat16*>(out), H, nsplit);
  return cudaGetLastError() == cudaSuccess ? 0 : RPEG_STATIC_ERR_LAUNCH;
}
