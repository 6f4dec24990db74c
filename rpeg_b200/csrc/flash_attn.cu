// Causal flash attention forward for sm_100a on packed variable-length sequences, head dim 128.
//
//   O = softmax(Q K^T * scale + causal) V      per (sequence, head)
//
// One CTA = one 128-row query tile of one head. Both GEMMs run on tcgen05 with accumulators in
// TMEM:
//   S = Q K^T   : A = Q tile, B = K tile, both K-major in shared memory (two 64-column 128B-swizzle
//                 atoms each), accumulator S in TMEM (double buffered so S_{j+1} is computed while
//                 the softmax of S_j runs);
//   O += P V    : A = P read directly from TMEM (bf16, written by the softmax threads into two P buffers of their
//                 own, TMEM columns 384..511), B = V tile in shared memory, MN-major (head dim contiguous).
// Softmax maps one thread to one query row (TMEM lane), so row max / row sum need no shuffles.
// The running max is only refreshed when it grows by more than 8 (in log2 units); a stale max is
// exact after the final division by l, and it makes the O rescale (TMEM load, scale, store) rare.
// That also makes the softmax ONE pass over S per tile: after the first tile the exponentials are taken against
// the current reference maximum while the same pass tracks the tile's true maximum; only when that maximum turns
// out more than 8 above the reference is O rescaled and the tile's P recomputed (S is still intact, because P has
// its own columns). TMEM loads run one chunk ahead of the arithmetic.
//
// Q/K/V are column blocks of one packed [T, ld] bf16 activation (the fused QKV projection output);
// cu_seqlens[b] is the first row of sequence b. Outputs: O [T, H*128] bf16, LSE [H, T] fp32.
//
// Replaces the reference's attention: Megatron core attention with an explicit (1,1,s,s) causal
// mask (RPEG/runtime/workers/megatron_worker.py:457,691,1618) / F.scaled_dot_product_attention in
// calibrate.py:230-376.
#include "common.cuh"
#include "rpeg_kernels.h"

namespace rpeg {

constexpr int FA_BM = 128;   // query rows per CTA
constexpr int FA_BN = 128;   // keys per tile
constexpr int FA_HD = 128;
constexpr int FA_THREADS = 192;
constexpr int FA_TILE_BYTES = 128 * 128 * 2;  // 32 KiB: one [128 x 128] bf16 tile (two 16 KiB atoms)
constexpr int FA_KV_STAGES = 2;
constexpr int FA_SMEM = FA_TILE_BYTES * (1 + 2 * FA_KV_STAGES) + 1024 + 256;
constexpr float FA_RESCALE_THRESHOLD = 8.0f;

// One softmax row pass over a 128-key tile held in TMEM (thread = query row). The four 32-column chunks are loaded
// one ahead of their use, so the TMEM load latency of chunk c+1 is covered by the arithmetic on chunk c.
//   row_max_pass : largest unscaled score of the row (masked keys excluded).
//   row_exp_pass : P = exp2(s * scale - m_ref) as packed bf16 into the P buffer, the row's sum of P added to `lsum`,
//                  and the largest unscaled score seen, so that one pass serves both the exponentials and the check
//                  whether m_ref was still a valid reference maximum.
template <bool MASK>
__device__ __forceinline__ float row_max_pass(uint32_t ts, int k0, int qi, int L) {
  uint32_t a[32], b[32];
  float tmax = -INFINITY;
  tmem_ld_32x32(ts, a);
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    tmem_wait_ld();
    uint32_t(&cur)[32] = (c & 1) ? b : a;
    if (c + 1 < 4) tmem_ld_32x32(ts + (c + 1) * 32, (c & 1) ? a : b);
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const int kj = k0 + c * 32 + i;
      if (!MASK || (kj <= qi && kj < L)) tmax = fmaxf(tmax, __uint_as_float(cur[i]));
    }
  }
  return tmax;
}

template <bool MASK>
__device__ __forceinline__ void row_exp_pass(uint32_t ts, uint32_t tp, float scale_log2, float m_ref, int k0, int qi, int L,
                                             bool row_valid, float& lsum, float& smax) {
  uint32_t a[32], b[32];
  tmem_ld_32x32(ts, a);
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    tmem_wait_ld();
    uint32_t(&cur)[32] = (c & 1) ? b : a;
    if (c + 1 < 4) tmem_ld_32x32(ts + (c + 1) * 32, (c & 1) ? a : b);
    uint32_t pk[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int kj = k0 + c * 32 + 2 * i;
      const float s0 = __uint_as_float(cur[2 * i]), s1 = __uint_as_float(cur[2 * i + 1]);
      float p0, p1;
      if (MASK) {
        const bool v0 = row_valid && kj <= qi && kj < L;
        const bool v1 = row_valid && kj + 1 <= qi && kj + 1 < L;
        if (v0) smax = fmaxf(smax, s0);
        if (v1) smax = fmaxf(smax, s1);
        p0 = v0 ? exp2f(fmaf(s0, scale_log2, -m_ref)) : 0.f;
        p1 = v1 ? exp2f(fmaf(s1, scale_log2, -m_ref)) : 0.f;
      } else {
        smax = fmaxf(smax, fmaxf(s0, s1));
        p0 = exp2f(fmaf(s0, scale_log2, -m_ref));
        p1 = exp2f(fmaf(s1, scale_log2, -m_ref));
      }
      lsum += p0 + p1;
      pk[i] = pack_bf16x2(p0, p1);
    }
    tmem_st_32x16(tp + c * 16, pk);
  }
}

__global__ void __launch_bounds__(FA_THREADS, 1)
flash_attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_qkv, const int* __restrict__ cu_seqlens,
                      __nv_bfloat16* __restrict__ out, float* __restrict__ lse_out, int T, int H, int Hkv,
                      int q_col0, int k_col0, int v_col0, float scale_log2, int* status) {
  const int b = blockIdx.z, h = blockIdx.y;
  const int qt = gridDim.x - 1 - blockIdx.x;  // heavy (late) tiles first
  const int seq0 = cu_seqlens[b];
  const int L = cu_seqlens[b + 1] - seq0;
  const int q0 = qt * FA_BM;
  if (q0 >= L) return;
  const int hk = h / (H / Hkv);
  const int kv_len = min(L, q0 + FA_BM);
  const int n_tiles = (kv_len + FA_BN - 1) / FA_BN;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_sm = smem;
  uint8_t* k_sm = smem + FA_TILE_BYTES;
  uint8_t* v_sm = k_sm + FA_KV_STAGES * FA_TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_sm + FA_KV_STAGES * FA_TILE_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = k_full + FA_KV_STAGES;
  uint64_t* v_full = k_empty + FA_KV_STAGES;
  uint64_t* v_empty = v_full + FA_KV_STAGES;
  uint64_t* s_full = v_empty + FA_KV_STAGES;  // [2]
  uint64_t* p_full = s_full + 2;              // [2]
  uint64_t* pv_done = p_full + 2;             // [2]: PV_j completes pv_done[j & 1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < FA_KV_STAGES; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) { mbar_init(&s_full[s], 1); mbar_init(&p_full[s], 4); }
    mbar_init(&pv_done[0], 1);
    mbar_init(&pv_done[1], 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 256;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmap_qkv);
      mbar_expect_tx(q_full, FA_TILE_BYTES);
      tma_load_2d(q_sm, &tmap_qkv, q_full, q_col0 + h * FA_HD, seq0 + q0);
      tma_load_2d(q_sm + 16384, &tmap_qkv, q_full, q_col0 + h * FA_HD + 64, seq0 + q0);
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j % FA_KV_STAGES;
        const uint32_t ph = static_cast<uint32_t>(j / FA_KV_STAGES) & 1u;
        if (!mbar_wait(&k_empty[st], ph ^ 1u, abort_flag, status, 500)) break;
        mbar_expect_tx(&k_full[st], FA_TILE_BYTES);
        tma_load_2d(k_sm + st * FA_TILE_BYTES, &tmap_qkv, &k_full[st], k_col0 + hk * FA_HD, seq0 + j * FA_BN);
        tma_load_2d(k_sm + st * FA_TILE_BYTES + 16384, &tmap_qkv, &k_full[st], k_col0 + hk * FA_HD + 64,
                    seq0 + j * FA_BN);
        if (!mbar_wait(&v_empty[st], ph ^ 1u, abort_flag, status, 501)) break;
        mbar_expect_tx(&v_full[st], FA_TILE_BYTES);
        tma_load_2d(v_sm + st * FA_TILE_BYTES, &tmap_qkv, &v_full[st], v_col0 + hk * FA_HD, seq0 + j * FA_BN);
        tma_load_2d(v_sm + st * FA_TILE_BYTES + 16384, &tmap_qkv, &v_full[st], v_col0 + hk * FA_HD + 64,
                    seq0 + j * FA_BN);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc_bf16(128, 128, 0, 1);
      const uint32_t q_addr = smem_u32(q_sm);
      auto issue_qk = [&](int j) {
        const int st = j % FA_KV_STAGES;
        const uint32_t k_addr = smem_u32(k_sm + st * FA_TILE_BYTES);
        const uint32_t ts = tmem_base + static_cast<uint32_t>((j & 1) * 128);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = static_cast<uint32_t>((k >> 2) * 16384 + (k & 3) * 32);
          umma_bf16_ss(ts, make_smem_desc_sw128(q_addr + off, 16, 1024), make_smem_desc_sw128(k_addr + off, 16, 1024),
                       idesc_qk, k != 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[st]);
        umma_commit(&s_full[j & 1]);
      };
      bool ok = mbar_wait(q_full, 0, abort_flag, status, 510);
      if (ok) ok = mbar_wait(&k_full[0], 0, abort_flag, status, 511);
      if (ok) {
        tc_fence_after_sync();
        issue_qk(0);
        for (int j = 0; j < n_tiles; ++j) {
          const int st = j % FA_KV_STAGES;
          const uint32_t ph = static_cast<uint32_t>(j / FA_KV_STAGES) & 1u;
          if (j + 1 < n_tiles) {
            const int st1 = (j + 1) % FA_KV_STAGES;
            const uint32_t ph1 = static_cast<uint32_t>((j + 1) / FA_KV_STAGES) & 1u;
            if (!mbar_wait(&k_full[st1], ph1, abort_flag, status, 512)) break;
            tc_fence_after_sync();
            issue_qk(j + 1);
          }
          if (!mbar_wait(&p_full[j & 1], static_cast<uint32_t>(j >> 1) & 1u, abort_flag, status, 513)) break;
          if (!mbar_wait(&v_full[st], ph, abort_flag, status, 514)) break;
          tc_fence_after_sync();
          const uint32_t v_addr = smem_u32(v_sm + st * FA_TILE_BYTES);
          const uint32_t tp = tmem_base + 384u + static_cast<uint32_t>((j & 1) * 64);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            // 16 keys per step: 8 packed TMEM columns of P, 16 rows (2 KiB) of the V tile.
            umma_bf16_ts(tmem_o, tp + k * 8, make_smem_desc_sw128(v_addr + k * 2048, 16384, 1024), idesc_pv,
                         (j | k) != 0 ? 1u : 0u);
          }
          umma_commit(&v_empty[st]);
          umma_commit(&pv_done[j & 1]);
        }
      }
    }
  } else {
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const int qi = q0 + r;  // position inside the sequence
    const bool row_valid = qi < L;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    // PV_j arrives on pv_done[j & 1], so each of the two barriers completes once per TWO tiles and its
    // completion number for PV_j is j >> 1. A parity wait is only right when the waiter is at most one
    // phase behind. That holds here: a warp that has seen s_full[j] knows every MMA issued before QK_j
    // has completed, PV_{j-2} and PV_{j-3} among them, and PV_{j+1} cannot be issued before this warp
    // has delivered P_{j+1}. So when it asks for PV_{j-1} (or, after the loop, for PV_{n-1}) the
    // barrier of that parity has finished either exactly the completions before the wanted one, or the
    // wanted one too. (With ONE barrier completing every tile a warp could be two phases behind and
    // then waited for a completion that needed its own next arrival.)
    auto wait_pv = [&](int tile, int where) -> bool {
      return __all_sync(0xffffffffu, mbar_wait(&pv_done[tile & 1], static_cast<uint32_t>(tile >> 1) & 1u, abort_flag,
                                               status, where));
    };
    for (int j = 0; j < n_tiles && ok; ++j) {
      const uint32_t ts = tmem_base + lane_base + static_cast<uint32_t>((j & 1) * 128);
      const uint32_t tp = tmem_base + lane_base + 384u + static_cast<uint32_t>((j & 1) * 64);
      if (!__all_sync(0xffffffffu, mbar_wait(&s_full[j & 1], static_cast<uint32_t>(j >> 1) & 1u, abort_flag, status, 520))) { ok = false; break; }
      tc_fence_after_sync();
      const int k0 = j * FA_BN;
      const bool need_mask = (k0 + FA_BN - 1 > q0) || (k0 + FA_BN > L);
      if (j == 0) {                       // no reference maximum yet: one extra pass finds it
        float t0 = need_mask ? row_max_pass<true>(ts, k0, qi, L) : row_max_pass<false>(ts, k0, qi, L);
        t0 *= scale_log2;                 // scale > 0, so max commutes with the scaling
        m_ref = (!row_valid || t0 == -INFINITY) ? 0.f : t0;
      }
      float lsum = 0.f, smax = -INFINITY;
      if (need_mask) row_exp_pass<true>(ts, tp, scale_log2, m_ref, k0, qi, L, row_valid, lsum, smax);
      else row_exp_pass<false>(ts, tp, scale_log2, m_ref, k0, qi, L, row_valid, lsum, smax);
      if (j > 0) {
        float tmax = smax * scale_log2;
        if (!row_valid || smax == -INFINITY) tmax = m_ref;
        const bool need = tmax > m_ref + FA_RESCALE_THRESHOLD;
        if (__any_sync(0xffffffffu, need)) {
          if (!wait_pv(j - 1, 521)) { ok = false; break; }
          tc_fence_after_sync();
          const float alpha = need ? exp2f(m_ref - tmax) : 1.f;
          if (need) { m_ref = tmax; l *= alpha; }
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t v[32];
            tmem_ld_32x32(tmem_o + lane_base + c * 32, v);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tmem_st_32x32(tmem_o + lane_base + c * 32, v);
          }
          // P of this tile again, against the new maximum (rows that kept theirs recompute the same values)
          lsum = 0.f;
          float unused = -INFINITY;
          if (need_mask) row_exp_pass<true>(ts, tp, scale_log2, m_ref, k0, qi, L, row_valid, lsum, unused);
          else row_exp_pass<false>(ts, tp, scale_log2, m_ref, k0, qi, L, row_valid, lsum, unused);
        }
      }
      l += lsum;
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[j & 1]);
    }
    if (ok && wait_pv(n_tiles - 1, 522)) {
      tc_fence_after_sync();
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* orow = out + (static_cast<size_t>(seq0 + qi) * H + h) * FA_HD;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_o + lane_base + c * 32, v);
        tmem_wait_ld();
        if (row_valid) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(v[i * 8 + 0]) * inv_l, __uint_as_float(v[i * 8 + 1]) * inv_l);
            o.y = pack_bf16x2(__uint_as_float(v[i * 8 + 2]) * inv_l, __uint_as_float(v[i * 8 + 3]) * inv_l);
            o.z = pack_bf16x2(__uint_as_float(v[i * 8 + 4]) * inv_l, __uint_as_float(v[i * 8 + 5]) * inv_l);
            o.w = pack_bf16x2(__uint_as_float(v[i * 8 + 6]) * inv_l, __uint_as_float(v[i * 8 + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow + c * 32 + i * 8) = o;
          }
        }
      }
      if (row_valid && lse_out != nullptr)
        lse_out[static_cast<size_t>(h) * T + seq0 + qi] = (m_ref + log2f(l)) * 0.6931471805599453f;
    }
  }

  __syncwarp();
  if (*abort_flag) __nanosleep(200000);
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

int make_tmap_bf16_2d(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer);

}  // namespace rpeg

using namespace rpeg;

extern "C" int rpeg_flash_attn_fwd(const void* qkv, int ld, int q_col0, int k_col0, int v_col0,
                                   const int* cu_seqlens, int B, int max_seqlen, int T, int H, int Hkv, int hd,
                                   float scale, void* out, float* lse, int* status, void* stream_v) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  if (hd != FA_HD || H % Hkv != 0) return -2;
  if ((ld | q_col0 | k_col0 | v_col0) & 7) return -3;
  if (reinterpret_cast<uintptr_t>(qkv) & 15) return -1;
  if (B <= 0 || T <= 0 || max_seqlen <= 0) return 0;
  CUtensorMap tm;
  const int rc = make_tmap_bf16_2d(&tm, qkv, static_cast<uint64_t>(ld), static_cast<uint64_t>(T),
                                   static_cast<uint64_t>(ld), 64, 128);
  if (rc) return rc;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(flash_attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FA_SMEM) != cudaSuccess)
      return -20;
    configured = true;
  }
  dim3 grid((max_seqlen + FA_BM - 1) / FA_BM, H, B);
  flash_attn_fwd_kernel<<<grid, FA_THREADS, FA_SMEM, stream>>>(tm, cu_seqlens, static_cast<__nv_bfloat16*>(out), lse,
                                                              T, H, Hkv, q_col0, k_col0, v_col0,
                                                              scale * 1.4426950408889634f, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

namespace rpeg {

// =====================================================================================
// Backward.
//
// One CTA owns one 128-key tile of one (sequence, head) and walks the query tiles at or below the
// diagonal. Everything is computed transposed (key = TMEM lane = thread) so that P^T and dS^T can
// feed the next MMA straight from TMEM:
//   S^T  = K Q^T          (A = K smem,  B = Q smem,  both K-major)      -> TMEM cols   0..127
//   dP^T = V dO^T         (A = V smem,  B = dO smem, both K-major)      -> TMEM cols 128..255
//   P^T  = exp2(S^T*scale - lse_q)            bf16, over S^T (cols 0..63)
//   dS^T = P^T * (dP^T - D_q)                 bf16, over dP^T (cols 128..191) and to shared memory
//   dV  += P^T  dO        (A = P^T TMEM,  B = dO smem read MN-major)    -> TMEM cols 256..383
//   dK  += dS^T Q         (A = dS^T TMEM, B = Q smem read MN-major)     -> TMEM cols 384..511
//   dQ_i = dS K           (A = dS^T smem read MN-major, B = K smem read MN-major)
//                                                                       -> TMEM cols 0..127 (S^T is dead)
// dQ_i is drained by the same threads (now lane = query row) into a [T, H*128] fp32 accumulator: every thread
// stages its row in shared memory, 64 columns at a time, and adds it to global memory with ONE bulk reduction
// (cp.reduce.async.bulk ... add.f32) per row and half, instead of 32 vector atomics per row (the atomics of all
// CTAs together saturated the L2's atomic rate and set the kernel's time). dK (scaled) and dV are written once
// at the end as bf16 into the K and V column blocks of a packed gradient buffer with the same layout as qkv.
// D_q = rowsum(dO * O) comes from a small pre-pass. Grouped-query attention (H a multiple of Hkv) is supported.
constexpr int FB_STAGE_ROW = 64 + 4;                       // floats per staged dQ row: 64 values + 16 bytes of padding
constexpr int FB_STAGE_BYTES = 128 * FB_STAGE_ROW * 4;     // (rows 272 bytes apart: conflict-free float4 stores)
constexpr int FB_SMEM = FA_TILE_BYTES * 5 + FB_STAGE_BYTES + 1024 + 1024 + 256;

// global[0 .. bytes) += shared[0 .. bytes) as fp32, one bulk operation in the current bulk group
__device__ __forceinline__ void bulk_reduce_add_f32(float* gdst, const float* ssrc, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(ssrc)),
               "r"(bytes)
               : "memory");
}

__global__ void attn_bwd_prep_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                     float* __restrict__ dvec, int T, int H) {
  // one warp per (token, head): D[h, t] = sum_d dO * O
  const long long w = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (w >= static_cast<long long>(T) * H) return;
  const int t = static_cast<int>(w / H), h = static_cast<int>(w % H);
  const int lane = threadIdx.x & 31;
  const size_t off = (static_cast<size_t>(t) * H + h) * FA_HD + lane * 4;
  const uint2 a = *reinterpret_cast<const uint2*>(o + off), b = *reinterpret_cast<const uint2*>(dout + off);
  const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), b0 = unpack_bf16x2(b.x), b1 = unpack_bf16x2(b.y);
  float s = a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y;
  s = warp_sum(s);
  if (lane == 0) dvec[static_cast<size_t>(h) * T + t] = s;
}

__global__ void __launch_bounds__(FA_THREADS, 1)
flash_attn_bwd_kernel(const __grid_constant__ CUtensorMap tmap_qkv, const __grid_constant__ CUtensorMap tmap_do,
                      const int* __restrict__ cu_seqlens, const float* __restrict__ lse,
                      const float* __restrict__ dvec, float* __restrict__ dq_acc,
                      __nv_bfloat16* __restrict__ dqkv, int ld_dqkv, int T, int H, int q_col0, int k_col0,
                      int v_col0, float scale, int Hkv, int* status) {
  // One CTA per (key tile, KV head, sequence). With grouped-query attention the G = H / Hkv query heads that
  // share this KV head are processed one after the other into the same dK / dV accumulators.
  const int b = blockIdx.z, hk = blockIdx.y, kt = blockIdx.x;  // early key tiles carry the most work
  const int G = H / Hkv;
  const int seq0 = cu_seqlens[b];
  const int L = cu_seqlens[b + 1] - seq0;
  const int k0 = kt * FA_BN;
  if (k0 >= L) return;
  const int n_qt = (L + FA_BM - 1) / FA_BM;
  const int n_iter = n_qt - kt;  // query tiles kt .. n_qt-1
  const int n_total = n_iter * G;  // flattened (query head of the group, query tile)
  const float scale_log2 = scale * 1.4426950408889634f;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* k_sm = smem;
  uint8_t* v_sm = k_sm + FA_TILE_BYTES;
  uint8_t* q_sm = v_sm + FA_TILE_BYTES;
  uint8_t* do_sm = q_sm + FA_TILE_BYTES;
  uint8_t* ds_sm = do_sm + FA_TILE_BYTES;
  float* dq_stage = reinterpret_cast<float*>(ds_sm + FA_TILE_BYTES);  // [128][FB_STAGE_ROW]
  float* lse_sm = dq_stage + 128 * FB_STAGE_ROW;                      // [128]
  float* d_sm = lse_sm + 128;                                       // [128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(d_sm + 128);
  uint64_t* kv_full = bars;         // K and V landed
  uint64_t* qdo_full = bars + 1;    // Q_i and dO_i landed
  uint64_t* qdo_empty = bars + 2;   // MMAs reading Q_i / dO_i / dS_i finished
  uint64_t* s_done = bars + 3;      // S^T and dP^T complete
  uint64_t* pds_ready = bars + 4;   // P^T and dS^T written (count 4)
  uint64_t* dq_done = bars + 5;     // dQ_i complete (implies dV, dK of this iteration too)
  uint64_t* dq_drained = bars + 6;  // dQ_i read out of TMEM (count 4)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 7);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1); mbar_init(qdo_full, 1); mbar_init(qdo_empty, 1); mbar_init(s_done, 1);
    mbar_init(pds_ready, 4); mbar_init(dq_done, 1); mbar_init(dq_drained, 4);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_s = tmem_base, t_dp = tmem_base + 128, t_dv = tmem_base + 256, t_dk = tmem_base + 384;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmap_qkv);
      tma_prefetch_desc(&tmap_do);
      mbar_expect_tx(kv_full, 2 * FA_TILE_BYTES);
      tma_load_2d(k_sm, &tmap_qkv, kv_full, k_col0 + hk * FA_HD, seq0 + k0);
      tma_load_2d(k_sm + 16384, &tmap_qkv, kv_full, k_col0 + hk * FA_HD + 64, seq0 + k0);
      tma_load_2d(v_sm, &tmap_qkv, kv_full, v_col0 + hk * FA_HD, seq0 + k0);
      tma_load_2d(v_sm + 16384, &tmap_qkv, kv_full, v_col0 + hk * FA_HD + 64, seq0 + k0);
      for (int it = 0; it < n_total; ++it) {
        const int h = hk * G + it / n_iter;
        const int q0 = (kt + it % n_iter) * FA_BM;
        if (!mbar_wait(qdo_empty, (static_cast<uint32_t>(it) & 1u) ^ 1u, abort_flag, status, 600)) break;
        mbar_expect_tx(qdo_full, 2 * FA_TILE_BYTES);
        tma_load_2d(q_sm, &tmap_qkv, qdo_full, q_col0 + h * FA_HD, seq0 + q0);
        tma_load_2d(q_sm + 16384, &tmap_qkv, qdo_full, q_col0 + h * FA_HD + 64, seq0 + q0);
        tma_load_2d(do_sm, &tmap_do, qdo_full, h * FA_HD, seq0 + q0);
        tma_load_2d(do_sm + 16384, &tmap_do, qdo_full, h * FA_HD + 64, seq0 + q0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t id_kk = make_idesc_bf16(128, 128, 0, 0);   // A K-major, B K-major
      constexpr uint32_t id_kmn = make_idesc_bf16(128, 128, 0, 1);  // A (TMEM or K-major), B MN-major
      constexpr uint32_t id_mnmn = make_idesc_bf16(128, 128, 1, 1); // both MN-major
      const uint32_t ka = smem_u32(k_sm), va = smem_u32(v_sm), qa = smem_u32(q_sm), da = smem_u32(do_sm),
                     dsa = smem_u32(ds_sm);
      bool ok = mbar_wait(kv_full, 0, abort_flag, status, 610);
      for (int it = 0; it < n_total && ok; ++it) {
        const uint32_t ph = static_cast<uint32_t>(it) & 1u;
        if (!mbar_wait(qdo_full, ph, abort_flag, status, 611)) break;
        if (it > 0 && !mbar_wait(dq_drained, ph ^ 1u, abort_flag, status, 612)) break;
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = static_cast<uint32_t>((k >> 2) * 16384 + (k & 3) * 32);
          umma_bf16_ss(t_s, make_smem_desc_sw128(ka + off, 16, 1024), make_smem_desc_sw128(qa + off, 16, 1024), id_kk,
                       k != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = static_cast<uint32_t>((k >> 2) * 16384 + (k & 3) * 32);
          umma_bf16_ss(t_dp, make_smem_desc_sw128(va + off, 16, 1024), make_smem_desc_sw128(da + off, 16, 1024), id_kk,
                       k != 0 ? 1u : 0u);
        }
        umma_commit(s_done);
        if (!mbar_wait(pds_ready, ph, abort_flag, status, 613)) break;
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < 8; ++k)  // dV += P^T dO : 16 queries per step
          umma_bf16_ts(t_dv, t_s + k * 8, make_smem_desc_sw128(da + k * 2048, 16384, 1024), id_kmn, (it | k) != 0 ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < 8; ++k)  // dK += dS^T Q
          umma_bf16_ts(t_dk, t_dp + k * 8, make_smem_desc_sw128(qa + k * 2048, 16384, 1024), id_kmn, (it | k) != 0 ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < 8; ++k)  // dQ = dS K : 16 keys per step, both operands MN-major
          umma_bf16_ss(t_s, make_smem_desc_sw128(dsa + k * 2048, 16384, 1024),
                       make_smem_desc_sw128(ka + k * 2048, 16384, 1024), id_mnmn, k != 0 ? 1u : 0u);
        umma_commit(qdo_empty);
        umma_commit(dq_done);
      }
    }
  } else {
    const int quad = warp & 3;
    const int r = quad * 32 + lane;  // key row inside the tile; later the query row when draining dQ
    const int kj = k0 + r;
    const bool key_valid = kj < L;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const int sm_tid = threadIdx.x - 64;  // 0..127
    bool ok = true;
    for (int it = 0; it < n_total && ok; ++it) {
      const uint32_t ph = static_cast<uint32_t>(it) & 1u;
      const int h = hk * G + it / n_iter;
      const int q0 = (kt + it % n_iter) * FA_BM;
      // per-query vectors of this tile (lse in log2 units); +inf lse turns invalid queries into p = 0
      {
        const int qi = q0 + sm_tid;
        const bool qv = qi < L;
        lse_sm[sm_tid] = qv ? lse[static_cast<size_t>(h) * T + seq0 + qi] * 1.4426950408889634f : INFINITY;
        d_sm[sm_tid] = qv ? dvec[static_cast<size_t>(h) * T + seq0 + qi] : 0.f;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (!__all_sync(0xffffffffu, mbar_wait(s_done, ph, abort_flag, status, 620))) { ok = false; break; }
      tc_fence_after_sync();
      const bool diag = (it % n_iter == 0);
      uint8_t* ds_row = ds_sm + r * 128;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t sv[32], dv[32];
        tmem_ld_32x32(t_s + lane_base + c * 32, sv);
        tmem_ld_32x32(t_dp + lane_base + c * 32, dv);
        tmem_wait_ld();
        uint32_t pp[16], dd[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float pv[2], gv[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int qq = c * 32 + 2 * i + e;  // query index inside the tile
            const bool valid = key_valid && (!diag || (q0 + qq >= kj));
            const float p = valid ? exp2f(__uint_as_float(sv[2 * i + e]) * scale_log2 - lse_sm[qq]) : 0.f;
            pv[e] = p;
            gv[e] = p * (__uint_as_float(dv[2 * i + e]) - d_sm[qq]);
          }
          pp[i] = pack_bf16x2(pv[0], pv[1]);
          dd[i] = pack_bf16x2(gv[0], gv[1]);
        }
        tmem_st_32x16(t_s + lane_base + c * 16, pp);
        tmem_st_32x16(t_dp + lane_base + c * 16, dd);
        // dS^T row r, queries [32c, 32c+32): atom c/2, 16-byte chunks (c%2)*4 .. +3, 128B swizzle
        uint8_t* atom = ds_row + (c >> 1) * 16384;
#pragma unroll
        for (int v4 = 0; v4 < 4; ++v4) {
          const int chunk = (c & 1) * 4 + v4;
          *reinterpret_cast<uint4*>(atom + ((chunk ^ (r & 7)) << 4)) =
              make_uint4(dd[v4 * 4 + 0], dd[v4 * 4 + 1], dd[v4 * 4 + 2], dd[v4 * 4 + 3]);
        }
      }
      tmem_wait_st();
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_ready);
      // drain dQ_i: lane = query row
      if (!__all_sync(0xffffffffu, mbar_wait(dq_done, ph, abort_flag, status, 621))) { ok = false; break; }
      tc_fence_after_sync();
      const int qi = q0 + r;
      float* dq_row = dq_acc + (static_cast<size_t>(seq0 + qi) * H + h) * FA_HD;
      float* my_stage = dq_stage + r * FB_STAGE_ROW;
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
        tma_store_wait_read<0>();                 // this thread's earlier bulk reads of its staging row are done
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(t_s + lane_base + (half * 2 + c) * 32, v);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 8; ++i)
            *reinterpret_cast<float4*>(my_stage + c * 32 + 4 * i) =
                make_float4(__uint_as_float(v[4 * i]) * scale, __uint_as_float(v[4 * i + 1]) * scale,
                            __uint_as_float(v[4 * i + 2]) * scale, __uint_as_float(v[4 * i + 3]) * scale);
        }
        fence_proxy_async_smem();                 // the row was written with ordinary stores, the bulk engine reads it
        if (qi < L) bulk_reduce_add_f32(dq_row + half * 64, my_stage, 64 * sizeof(float));
        tma_store_commit();
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(dq_drained);
    }
    tma_store_wait<0>();          // every bulk reduction of this thread has been performed
    if (ok) {
      // dq_done of the last iteration also covers the last dV / dK accumulation
      tc_fence_after_sync();
      __nv_bfloat16* dk_row = dqkv + static_cast<size_t>(seq0 + kj) * ld_dqkv + k_col0 + hk * FA_HD;
      __nv_bfloat16* dv_row = dqkv + static_cast<size_t>(seq0 + kj) * ld_dqkv + v_col0 + hk * FA_HD;
#pragma unroll 1
      for (int c = 0; c < 8; ++c) {
        uint32_t v[32];
        const bool is_k = c >= 4;
        tmem_ld_32x32((is_k ? t_dk : t_dv) + lane_base + (c & 3) * 32, v);
        tmem_wait_ld();
        if (key_valid) {
          const float sc = is_k ? scale : 1.f;
          __nv_bfloat16* dst = (is_k ? dk_row : dv_row) + (c & 3) * 32;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(v[i * 8 + 0]) * sc, __uint_as_float(v[i * 8 + 1]) * sc);
            o.y = pack_bf16x2(__uint_as_float(v[i * 8 + 2]) * sc, __uint_as_float(v[i * 8 + 3]) * sc);
            o.z = pack_bf16x2(__uint_as_float(v[i * 8 + 4]) * sc, __uint_as_float(v[i * 8 + 5]) * sc);
            o.w = pack_bf16x2(__uint_as_float(v[i * 8 + 6]) * sc, __uint_as_float(v[i * 8 + 7]) * sc);
            *reinterpret_cast<uint4*>(dst + i * 8) = o;
          }
        }
        __syncwarp();
      }
    }
  }

  __syncwarp();
  if (*abort_flag) __nanosleep(200000);
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// dq (bf16, Q column block of dqkv) <- dq_acc (fp32 [T, H*128])
__global__ void dq_store_kernel(const float* __restrict__ dq_acc, __nv_bfloat16* __restrict__ dqkv, int ld, int q_col0,
                                int T, int width) {
  const int wv = width >> 2;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<long long>(T) * wv) return;
  const int t = static_cast<int>(idx / wv), j = static_cast<int>(idx % wv);
  const float4 a = reinterpret_cast<const float4*>(dq_acc + static_cast<size_t>(t) * width)[j];
  uint2 o;
  o.x = pack_bf16x2(a.x, a.y);
  o.y = pack_bf16x2(a.z, a.w);
  *reinterpret_cast<uint2*>(dqkv + static_cast<size_t>(t) * ld + q_col0 + j * 4) = o;
}

}  // namespace rpeg (reopened below for the launcher)

// qkv/out/lse are the forward's tensors; dout is [T, H*128] bf16. dq_acc is a caller-provided
// fp32 [T, H*128] scratch that this call zeroes. dqkv ([T, ld_dqkv] bf16) receives dQ, dK, dV in
// the same column blocks as qkv.
extern "C" int rpeg_flash_attn_bwd(const void* qkv, int ld, int q_col0, int k_col0, int v_col0, const void* out,
                                   const void* dout, const float* lse, const int* cu_seqlens, int B,
                                   int max_seqlen, int T, int H, int Hkv, int hd, float scale, float* dvec,
                                   float* dq_acc, void* dqkv, int ld_dqkv, int* status, void* stream_v) {
  using namespace rpeg;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  if (hd != FA_HD || Hkv <= 0 || H % Hkv != 0) return -2;
  if ((ld | ld_dqkv | q_col0 | k_col0 | v_col0) & 7) return -3;
  if ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(dout)) & 15) return -1;
  if (B <= 0 || T <= 0 || max_seqlen <= 0) return 0;
  CUtensorMap tm_qkv, tm_do;
  int rc = make_tmap_bf16_2d(&tm_qkv, qkv, static_cast<uint64_t>(ld), static_cast<uint64_t>(T), static_cast<uint64_t>(ld), 64, 128);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tm_do, dout, static_cast<uint64_t>(H) * FA_HD, static_cast<uint64_t>(T),
                         static_cast<uint64_t>(H) * FA_HD, 64, 128);
  if (rc) return rc - 100;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(flash_attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FB_SMEM) != cudaSuccess)
      return -20;
    configured = true;
  }
  const long long warps = static_cast<long long>(T) * H;
  attn_bwd_prep_kernel<<<static_cast<unsigned>((warps * 32 + 255) / 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(dout), dvec, T, H);
  if (cudaMemsetAsync(dq_acc, 0, static_cast<size_t>(T) * H * FA_HD * sizeof(float), stream) != cudaSuccess) return -22;
  dim3 grid((max_seqlen + FA_BN - 1) / FA_BN, Hkv, B);
  flash_attn_bwd_kernel<<<grid, FA_THREADS, FB_SMEM, stream>>>(tm_qkv, tm_do, cu_seqlens, lse, dvec, dq_acc,
                                                              static_cast<__nv_bfloat16*>(dqkv), ld_dqkv, T, H, q_col0,
                                                              k_col0, v_col0, scale, Hkv, status);
  const long long n = static_cast<long long>(T) * (H * FA_HD / 4);
  dq_store_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(dq_acc, static_cast<__nv_bfloat16*>(dqkv),
                                                                             ld_dqkv, q_col0, T, H * FA_HD);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}
