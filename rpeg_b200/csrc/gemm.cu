// bf16 GEMM for sm_100a: TMA -> shared memory -> tcgen05.mma -> TMEM -> epilogue.
//
//   C[M,N] = op(A)[M,K] * op(B)[N,K]^T        (fp32 accumulate in TMEM)
//
// transA = 0: A is stored [M,K] (K contiguous, "K-major");  1: A is stored [K,M] ("MN-major").
// transB = 0: B is stored [N,K] (the [out,in] layout of a linear weight); 1: B is stored [K,N].
// Those four combinations cover forward (x W^T), dgrad (dy W) and wgrad (dy^T x) of a linear layer
// without materialising a transposed copy: the MN-major cases only change the TMA box and the
// shared-memory matrix descriptor.
//
// Kernel structure (persistent, one CTA per SM, 192 threads):
//   warp 0      TMA producer: fills a ring of STAGES {A tile, B tile} buffers
//   warp 1      allocates TMEM, issues tcgen05.mma from one thread, frees TMEM at the end
//   warps 2..5  epilogue: tcgen05.ld the 128 x BN fp32 accumulator (thread = row), convert, store
// The accumulator is double buffered in TMEM (2 x BN columns) so the epilogue of tile i overlaps
// the main loop of tile i+1.
//
// Replaces the cuBLASLt / TransformerEngine GEMMs the reference reaches through megatron-core
// (reference: RPEG/runtime/workers/megatron_worker.py:676-715 builds the GPTModel whose
// linear_qkv / linear_proj / linear_fc1 / linear_fc2 / output_layer run them).
#include <cstdlib>
#include "common.cuh"
#include "rpeg_kernels.h"

namespace rpeg {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = one 128-byte swizzle row
constexpr int GEMM_THREADS = 192;
constexpr int SMEM_BUDGET = 227 * 1024 - 2048;

// AR: rows of the A tile that exist in shared memory (128 in every instantiation in use). A variant with AR = 32 for
// decode GEMMs of up to 32 rows (6 stages of 256-wide weight tiles instead of 4) measured 5 % SLOWER per decode step:
// the streaming rate of the skinny GEMMs is not limited by the bytes in flight per SM.
template <int BN, int AR = BM>
struct GemmCfg {
  static constexpr int A_BYTES = AR * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES_RAW = SMEM_BUDGET / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 10 ? 10 : STAGES_RAW;
  static constexpr int TMEM_COLS = (2 * BN) < 32 ? 32 : (2 * BN);
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 512 /*barriers*/;
};

// EPI_SWIGLU: B is a gated-MLP weight [2f, K] (gate rows, then up rows). Output tile tn covers the activation columns
// [128 tn, 128 tn + 128): its B tile is 128 gate rows stacked on the 128 up rows of the same columns, the accumulator
// holds gate in columns 0..127 and up in 128..255, and the epilogue stores silu(gate) * up as bf16, so the
// [M, 2f] pre-activation never goes to memory (N is f here, BN must be 256).
enum { EPI_BF16 = 0, EPI_F32 = 1, EPI_SWIGLU = 2 };

// Optional gate in front of the first operand load: `n` version words (written by the GPUs that push new weights
// into B's buffer, system-scope release) must all have reached `min_version` before any tile of this GEMM is
// read. The wait is bounded by `timeout_ns`; on expiry the kernel records RPEG_ERR_FLAG_TIMEOUT and drains.
struct WeightGate {
  const unsigned* flags;
  int n;
  unsigned min_version;
  unsigned long long timeout_ns;
};

template <int BN, int EPI, bool A_MN, bool B_MN, int AR = BM>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                         void* __restrict__ Cout, int M, int N, int K, int ldc, int accumulate, int k_splits,
                         long long split_stride, int* status, WeightGate gate, int pdl, int a_rows) {
  using Cfg = GemmCfg<BN, AR>;
  // K-major A with few rows (decode): the TMA box covers only `a_rows` rows of the 128-row A tile. The MMA still reads
  // 128 rows; what it computes from the rows nobody loaded lands in accumulator rows that the epilogue never stores.
  const uint32_t stage_tx = static_cast<uint32_t>(Cfg::B_BYTES + (A_MN ? Cfg::A_BYTES : a_rows * BK * 2));
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* bar_area = smem + STAGES * Cfg::STAGE_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(bar_area);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr int TN = (EPI == EPI_SWIGLU) ? BN / 2 : BN;   // output columns per tile
  const int m_tiles = (M + BM - 1) / BM;
  const int n_tiles = (N + TN - 1) / TN;
  const int num_tiles = m_tiles * n_tiles;
  const int num_kb = (K + BK - 1) / BK;
  // Split-K: work item w = tile * k_splits + split; a split covers kb_per consecutive K blocks and
  // writes its own fp32 partial at Cout + split * split_stride.
  const int kb_per = (num_kb + k_splits - 1) / k_splits;
  const int num_items = num_tiles * k_splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], 4);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // Launched as a programmatic dependent (decode: B is a weight matrix that no kernel of the step writes): the
  // set-up above already ran under the previous kernel's tail, and the producer streams the first weight tiles
  // before it waits for that kernel; every other thread waits here, before it can touch A, C or the workspace.
  if (pdl) {
    griddep_launch();
    if (threadIdx.x != 0) griddep_wait();
  }

  // Tile order: groups of 8 M-tiles sweep N together so the A rows stay in L2.
  constexpr int GROUP_M = 8;
  auto tile_coords = [&](int t, int& tm, int& tn) {
    const int per_group = GROUP_M * n_tiles;
    const int g = t / per_group;
    const int first_m = g * GROUP_M;
    const int gsize = min(m_tiles - first_m, GROUP_M);
    const int r = t - g * per_group;
    tm = first_m + (r % gsize);
    tn = r / gsize;
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int skip = 0;                      // k-blocks of the first item that the early weight prefetch already issued
      if (gate.flags != nullptr) {
        const uint64_t t0 = global_timer_ns();
        for (int i = 0; i < gate.n; ++i) {
          for (;;) {
            unsigned seen;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(gate.flags + i) : "memory");
            if (static_cast<int>(seen - gate.min_version) >= 0) break;
            if (global_timer_ns() - t0 > gate.timeout_ns) {
              record_error(status, RPEG_ERR_FLAG_TIMEOUT, 150, i);
              *abort_flag = 1;
              goto producer_done;
            }
            __nanosleep(500);
          }
        }
        // the new weights were written with ordinary (peer) stores; the loads below go through the async proxy
        asm volatile("fence.proxy.async.global;" ::: "memory");
      }
      if (pdl) {
        if constexpr (!A_MN && !B_MN) {
          if (static_cast<int>(blockIdx.x) < num_items) {
            int tm, tn;
            tile_coords(blockIdx.x / k_splits, tm, tn);
            const int kb0 = (blockIdx.x % k_splits) * kb_per, kb1 = min(num_kb, kb0 + kb_per);
            const int pre = min(STAGES, kb1 - kb0);
            for (int i = 0; i < pre; ++i) {            // weights first: they do not depend on the previous kernel
              mbar_expect_tx(&full_bar[i], stage_tx);
              tma_load_2d(smem + i * Cfg::STAGE_BYTES + Cfg::A_BYTES, &tmap_b, &full_bar[i], (kb0 + i) * BK, tn * BN);  // never EPI_SWIGLU
            }
            griddep_wait();
            for (int i = 0; i < pre; ++i)
              tma_load_2d(smem + i * Cfg::STAGE_BYTES, &tmap_a, &full_bar[i], (kb0 + i) * BK, tm * BM);
            skip = pre;
            if (pre == STAGES) phase = 1u; else stage = pre;
          } else {
            griddep_wait();
          }
        } else {
          griddep_wait();
        }
      }
      for (int w = blockIdx.x; w < num_items; w += gridDim.x) {
        int tm, tn;
        tile_coords(w / k_splits, tm, tn);
        const int m0 = tm * BM, n0 = tn * TN;
        const int kb0 = (w % k_splits) * kb_per, kb1 = min(num_kb, kb0 + kb_per);
        const int kb_first = kb0 + skip;
        skip = 0;
        for (int kb = kb_first; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, status, 100)) goto producer_done;
          uint8_t* sa = smem + stage * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          mbar_expect_tx(&full_bar[stage], stage_tx);
          if constexpr (!A_MN) {
            tma_load_2d(sa, &tmap_a, &full_bar[stage], kb * BK, m0);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_2d(sa + c * (64 * BK * 2), &tmap_a, &full_bar[stage], m0 + c * 64, kb * BK);
          }
          if constexpr (EPI == EPI_SWIGLU) {
            // gate rows n0.. and up rows N + n0.. (N = f): two boxes of BN / 2 rows, stacked in the B tile
            tma_load_2d(sb, &tmap_b, &full_bar[stage], kb * BK, n0);
            tma_load_2d(sb + (BN / 2) * BK * 2, &tmap_b, &full_bar[stage], kb * BK, N + n0);
          } else if constexpr (!B_MN) {
            tma_load_2d(sb, &tmap_b, &full_bar[stage], kb * BK, n0);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sb + c * (64 * BK * 2), &tmap_b, &full_bar[stage], n0 + c * 64, kb * BK);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    producer_done:;
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int buf = 0;
      uint32_t acc_phase = 0;
      for (int w = blockIdx.x; w < num_items; w += gridDim.x) {
        if (!mbar_wait(&tempty_bar[buf], acc_phase ^ 1u, abort_flag, status, 200)) goto mma_done;
        tc_fence_after_sync();
        const uint32_t tacc = tmem_base + static_cast<uint32_t>(buf * BN);
        const int kb0 = (w % k_splits) * kb_per, kb1 = min(num_kb, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, status, 201)) goto mma_done;
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * Cfg::STAGE_BYTES);
          const uint32_t sb = sa + Cfg::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // K-major: 16 bf16 along K = 32 bytes inside the swizzle row.
            // MN-major: 16 K rows of 128 bytes; 64-element MN chunks are one TMA box (8 KiB) apart.
            const uint64_t da = A_MN ? make_smem_desc_sw128(sa + k * 2048, 64 * BK * 2, 1024)
                                     : make_smem_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc_sw128(sb + k * 2048, 64 * BK * 2, 1024)
                                     : make_smem_desc_sw128(sb + k * 32, 16, 1024);
            umma_bf16_ss(tacc, da, db, idesc, (kb > kb0 || k != 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        umma_commit(&tfull_bar[buf]);
        if (++buf == 2) { buf = 0; acc_phase ^= 1u; }
      }
    mma_done:;
    }
  } else {
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    int buf = 0;
    uint32_t acc_phase = 0;
    for (int w = blockIdx.x; w < num_items; w += gridDim.x) {
      int tm, tn;
      tile_coords(w / k_splits, tm, tn);
      const long long split_off = static_cast<long long>(w % k_splits) * split_stride;
      const int row = tm * BM + quad * 32 + lane;
      const int n0 = tn * TN;
      if (!__all_sync(0xffffffffu, mbar_wait(&tfull_bar[buf], acc_phase, abort_flag, status, 300))) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(buf * BN);
      if constexpr (EPI == EPI_SWIGLU) {
#pragma unroll 1
        for (int c = 0; c < TN / 32; ++c) {
          uint32_t gv[32], uv[32];
          tmem_ld_32x32(taddr + c * 32, gv);
          tmem_ld_32x32(taddr + TN + c * 32, uv);
          tmem_wait_ld();
          const int col0 = n0 + c * 32;
          if (row < M && col0 < N) {
            __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(Cout) + static_cast<size_t>(row) * ldc + col0;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              if (col0 + v * 8 < N) {
                uint32_t o[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float g0 = __uint_as_float(gv[v * 8 + 2 * e]), g1 = __uint_as_float(gv[v * 8 + 2 * e + 1]);
                  const float a0 = g0 / (1.f + __expf(-g0)) * __uint_as_float(uv[v * 8 + 2 * e]);
                  const float a1 = g1 / (1.f + __expf(-g1)) * __uint_as_float(uv[v * 8 + 2 * e + 1]);
                  o[e] = pack_bf16x2(a0, a1);
                }
                *reinterpret_cast<uint4*>(crow + v * 8) = make_uint4(o[0], o[1], o[2], o[3]);
              }
            }
          }
        }
      } else
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_wait_ld();
        const int col0 = n0 + c * 32;
        if (row < M && col0 < N) {
          if constexpr (EPI == EPI_BF16) {
            __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(Cout) + static_cast<size_t>(row) * ldc + col0;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              if (col0 + v * 8 < N) {
                uint4 o;
                o.x = pack_bf16x2(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]));
                o.y = pack_bf16x2(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
                o.z = pack_bf16x2(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
                o.w = pack_bf16x2(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
                *reinterpret_cast<uint4*>(crow + v * 8) = o;
              }
            }
          } else {
            float* crow = reinterpret_cast<float*>(Cout) + split_off + static_cast<size_t>(row) * ldc + col0;
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              if (col0 + v * 4 < N) {
                float4 o = make_float4(__uint_as_float(r[v * 4 + 0]), __uint_as_float(r[v * 4 + 1]),
                                       __uint_as_float(r[v * 4 + 2]), __uint_as_float(r[v * 4 + 3]));
                if (accumulate) {
                  const float4 p = *reinterpret_cast<const float4*>(crow + v * 4);
                  o.x += p.x; o.y += p.y; o.z += p.z; o.w += p.w;
                }
                *reinterpret_cast<float4*>(crow + v * 4) = o;
              }
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[buf]);
      if (++buf == 2) { buf = 0; acc_phase ^= 1u; }
    }
  }

  // Teardown. After an aborted wait there may be bulk copies in flight into this CTA's shared
  // memory; give them time to land before the block exits.
  __syncwarp();
  if (*abort_flag) __nanosleep(200000);
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------- host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D bf16 tensor map: `inner` contiguous elements, `outer` rows of `ld` elements, 128-byte swizzle.
int make_tmap_bf16_2d(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -10;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -11;
}

template <int BN, int EPI, bool A_MN, bool B_MN, int AR = BM>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, void* C, int M, int N, int K, int ldc,
                       int accumulate, int k_splits, long long split_stride, int* status, int num_sms,
                       cudaStream_t stream, WeightGate gate = WeightGate{nullptr, 0, 0u, 0ull}, int pdl = 0, int a_rows = BM) {
  using Cfg = GemmCfg<BN, AR>;
  auto kern = gemm_bf16_tcgen05_kernel<BN, EPI, A_MN, B_MN, AR>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return -20;
    configured = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN) * k_splits;
  const int grid = tiles < num_sms ? tiles : num_sms;
  if (pdl) {
    // programmatic dependent launch: this grid may be scheduled while the previous kernel of the stream drains
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, ta, tb, C, M, N, K, ldc, accumulate, k_splits, split_stride, status, gate, 1, a_rows) == cudaSuccess
               ? 0 : -21;
  }
  kern<<<grid, GEMM_THREADS, Cfg::SMEM_BYTES, stream>>>(ta, tb, C, M, N, K, ldc, accumulate, k_splits, split_stride,
                                                        status, gate, 0, a_rows);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

template <int BN, int EPI>
static int dispatch_major(int transA, int transB, const CUtensorMap& ta, const CUtensorMap& tb, void* C, int M,
                          int N, int K, int ldc, int accumulate, int k_splits, long long split_stride, int* status,
                          int num_sms, cudaStream_t stream, WeightGate gate = WeightGate{nullptr, 0, 0u, 0ull}, int pdl = 0, int a_rows = BM) {
  if (!transA && !transB) return launch_gemm<BN, EPI, false, false>(ta, tb, C, M, N, K, ldc, accumulate, k_splits, split_stride, status, num_sms, stream, gate, pdl, a_rows);
  if (transA && !transB) return launch_gemm<BN, EPI, true, false>(ta, tb, C, M, N, K, ldc, accumulate, k_splits, split_stride, status, num_sms, stream, gate, pdl, a_rows);
  if constexpr (BN >= 64) {  // an MN-major B tile is built from 64-column TMA boxes
    if (!transA) return launch_gemm<BN, EPI, false, true>(ta, tb, C, M, N, K, ldc, accumulate, k_splits, split_stride, status, num_sms, stream, gate, pdl, a_rows);
    return launch_gemm<BN, EPI, true, true>(ta, tb, C, M, N, K, ldc, accumulate, k_splits, split_stride, status, num_sms, stream, gate, pdl, a_rows);
  }
  return -30;
}

static int g_num_sms = 0;


}  // namespace rpeg

using namespace rpeg;

// Rows of A that the TMA box fetches per k-block: the whole 128-row tile, or only 32 / 64 rows when the problem has no
// more (decode). Per k-block an SM then takes in 36 or 40 KB instead of 48 KB for a 256-wide weight tile, which is what
// counts when the weights stream from memory and the activation tile is re-read from L2 by every CTA.
// RPEG_GEMM_SKINNY_A=0 keeps the full box.
static int a_box_rows(int M, int transA) {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("RPEG_GEMM_SKINNY_A");
    on = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  if (transA || !on) return BM;
  return M <= 32 ? 32 : (M <= 64 ? 64 : BM);
}

static int gemm_impl(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int transA,
                     int transB, int out_fp32, int accumulate, int bn_hint, float* workspace, long long workspace_elems,
                     int* status, void* stream_v, WeightGate gate);

extern "C" int rpeg_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb,
                              int ldc, int transA, int transB, int out_fp32, int accumulate, int bn_hint,
                              float* workspace, long long workspace_elems, int* status, void* stream_v) {
  return gemm_impl(A, B, C, M, N, K, lda, ldb, ldc, transA, transB, out_fp32, accumulate, bn_hint, workspace,
                   workspace_elems, status, stream_v, WeightGate{nullptr, 0, 0u, 0ull});
}

// The same GEMM behind a weight-version gate: no operand tile is loaded before gate_flags[0..gate_words) have all
// reached min_version (see WeightGate). The first GEMM of a generation phase uses it on the weight buffer that
// the training ranks push into, so waiting for the push and the first use of the weights are one launch. The
// in-kernel wait is capped at 1.5 s (below the pipeline's own wait limit); longer waits belong on the host.
extern "C" int rpeg_gemm_bf16_gated(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb,
                                    int ldc, int transA, int transB, int out_fp32, int accumulate, int bn_hint,
                                    float* workspace, long long workspace_elems, const unsigned* gate_flags,
                                    int gate_words, unsigned min_version, unsigned long long timeout_ns, int* status,
                                    void* stream_v) {
  if (gate_flags == nullptr || gate_words < 1) return -6;
  const unsigned long long cap = 1500000000ull;
  return gemm_impl(A, B, C, M, N, K, lda, ldb, ldc, transA, transB, out_fp32, accumulate, bn_hint, workspace,
                   workspace_elems, status, stream_v,
                   WeightGate{gate_flags, gate_words, min_version, timeout_ns < cap ? timeout_ns : cap});
}

static int gemm_impl(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int transA,
                     int transB, int out_fp32, int accumulate, int bn_hint, float* workspace, long long workspace_elems,
                     int* status, void* stream_v, WeightGate gate) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  // TMA needs 16-byte aligned bases and row pitches; the vector epilogue needs N and ldc % 8 == 0.
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15) return -1;
  if ((lda | ldb | ldc) & 7) return -2;
  if (N & 7) return -3;
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  // bit 0x1000 of the tile-width hint: the caller chains this GEMM into a decode step (see `pdl` below)
  const bool chain = (bn_hint & 0x1000) != 0;
  bn_hint &= 0xfff;
  int bn = bn_hint;
  if (bn == 0) {
    const int m_tiles = (M + BM - 1) / BM;
    bn = 256;
    // Few M tiles (decode, small batches): shrink BN until the grid covers the SMs so the weight
    // stream is pulled by every SM.
    while (bn > 32 && m_tiles * ((N + bn - 1) / bn) < g_num_sms) bn >>= 1;
    if (transB && bn < 64) bn = 64;
  }
  // Split-K for skinny problems (decode): when one wave of output tiles leaves most SMs idle, cut
  // K so every SM streams a slice of the weights; fp32 partials go to `workspace` and a second
  // kernel sums them into the bf16 output.
  int k_splits = 1;
  long long split_stride = 0;
  void* gemm_out = C;
  int gemm_ldc = ldc, gemm_fp32 = out_fp32;
  if (workspace != nullptr && !out_fp32 && !accumulate && M <= 2 * BM) {
    if (bn_hint == 0) bn = N >= 256 ? 256 : (N >= 128 ? 128 : (N >= 64 ? 64 : 32));
    const int tiles = ((M + BM - 1) / BM) * ((N + bn - 1) / bn);
    const int num_kb = (K + BK - 1) / BK;
    // Pick the split count by a small cost model in units of "K blocks streamed by one CTA":
    // waves * blocks per item (+2 per wave for pipeline fill and drain) + the fp32 partial traffic
    // (written by the GEMM, read by the reduction) spread over all SMs.
    const long long per_split = static_cast<long long>(M) * N;
    const double block_bytes = static_cast<double>(g_num_sms) * BK * (bn + BM) * 2.0;
    int want = 1;
    double best = 1e30;
    const int max_s = num_kb / 2 > 32 ? 32 : num_kb / 2;
    for (int sp = 1; sp <= (max_s < 1 ? 1 : max_s); ++sp) {
      const int kb_per = (num_kb + sp - 1) / sp;
      const int real = (num_kb + kb_per - 1) / kb_per;
      if (real != sp) continue;
      if (sp > 1 && per_split > 0 && workspace_elems / per_split < sp) break;
      const int waves = (tiles * sp + g_num_sms - 1) / g_num_sms;
      const double cost = waves * (kb_per + 2.0) + (sp > 1 ? sp * per_split * 8.0 / block_bytes : 0.0);
      if (cost < best - 1e-9) { best = cost; want = sp; }
    }
    if (want > 1) {
      const int kb_per = (num_kb + want - 1) / want;
      k_splits = (num_kb + kb_per - 1) / kb_per;
      split_stride = per_split;
      gemm_out = workspace;
      gemm_ldc = N;
      gemm_fp32 = 1;
    }
  }
  // Decode GEMMs (the caller passes the split-K workspace): activation x weight^T, and no kernel of a decode step
  // writes the weights, so the grid may start under the previous kernel's tail and prefetch weight tiles.
  const int pdl = ((workspace != nullptr || chain) && !transA && !transB && !accumulate && gate.flags == nullptr) ? pdl_enabled() : 0;
  CUtensorMap ta, tb;
  int rc;
  const int a_rows = a_box_rows(M, transA);
  if (!transA) rc = make_tmap_bf16_2d(&ta, A, K, M, lda, BK, a_rows);
  else rc = make_tmap_bf16_2d(&ta, A, M, K, lda, 64, BK);
  if (rc) return rc;
  if (!transB) rc = make_tmap_bf16_2d(&tb, B, K, N, ldb, BK, bn);
  else rc = make_tmap_bf16_2d(&tb, B, N, K, ldb, 64, BK);
  if (rc) return rc - 100;
#define RPEG_GEMM_CASE(BN_)                                                                                      \
  case BN_:                                                                                                       \
    rc = gemm_fp32 ? dispatch_major<BN_, EPI_F32>(transA, transB, ta, tb, gemm_out, M, N, K, gemm_ldc, accumulate, \
                                                  k_splits, split_stride, status, g_num_sms, stream, gate, pdl, a_rows)   \
                   : dispatch_major<BN_, EPI_BF16>(transA, transB, ta, tb, gemm_out, M, N, K, gemm_ldc, accumulate, \
                                                   k_splits, split_stride, status, g_num_sms, stream, gate, pdl, a_rows); \
    break;
  switch (bn) {
    RPEG_GEMM_CASE(256)
    RPEG_GEMM_CASE(128)
    RPEG_GEMM_CASE(64)
    RPEG_GEMM_CASE(32)
    default:
      return -4;
  }
#undef RPEG_GEMM_CASE
  if (rc == 0 && k_splits > 1) rc = rpeg_splitk_reduce(workspace, C, M, N, ldc, k_splits, stream_v);
  return rc;
}


// act[M, f] = silu(A W_gate^T) * (A W_up^T) with W = [W_gate; W_up] stored [2f, K] (the gated MLP's first linear with
// its activation in the GEMM epilogue). f must be a multiple of 128; A [M, K] and W rows K-contiguous.
extern "C" int rpeg_gemm_swiglu(const void* A, const void* W, void* C, int M, int f, int K, int lda, int ldw, int ldc,
                                int* status, void* stream_v) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  if (M <= 0 || f <= 0 || K <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(C)) & 15) return -1;
  if ((lda | ldw | ldc) & 7) return -2;
  if (f % 128) return -3;
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  CUtensorMap ta, tb;
  int rc = make_tmap_bf16_2d(&ta, A, K, M, lda, BK, BM);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tb, W, K, 2ull * f, ldw, BK, 128);
  if (rc) return rc - 100;
  using Cfg = GemmCfg<256>;
  auto kern = gemm_bf16_tcgen05_kernel<256, EPI_SWIGLU, false, false>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess) return -20;
    configured = true;
  }
  const int tiles = ((M + BM - 1) / BM) * (f / 128);
  const int grid = tiles < g_num_sms ? tiles : g_num_sms;
  kern<<<grid, GEMM_THREADS, Cfg::SMEM_BYTES, stream>>>(ta, tb, C, M, f, K, ldc, 0, 1, 0, status, WeightGate{nullptr, 0, 0u, 0ull}, 0, BM);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

// Skinny GEMM that leaves its split-K partials for the consumer: C_s[M,N] (fp32, s = 0..splits-1, `M*N`
// apart in `workspace`) with sum_s C_s = A[M,K] * B[N,K]^T. The split count is chosen by the same cost
// model as rpeg_gemm_bf16 and returned in *k_splits_out; kernels that read the result (RMSNorm, SwiGLU,
// RoPE + KV append for decode) add the partials while they load them, so the separate reduction pass
// and its round trip through memory disappear.
extern "C" int rpeg_gemm_bf16_partials(const void* A, const void* B, int M, int N, int K, int lda, int ldb,
                                       float* workspace, long long workspace_elems, int* k_splits_out, int* status,
                                       void* stream_v) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  if (k_splits_out == nullptr || workspace == nullptr) return -5;
  *k_splits_out = 1;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(workspace)) & 15) return -1;
  if ((lda | ldb) & 7) return -2;
  if (N & 7) return -3;
  const long long per_split = static_cast<long long>(M) * N;
  if (workspace_elems < per_split) return -6;
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int bn = N >= 256 ? 256 : (N >= 128 ? 128 : (N >= 64 ? 64 : 32));
  const int tiles = ((M + BM - 1) / BM) * ((N + bn - 1) / bn);
  const int num_kb = (K + BK - 1) / BK;
  const double block_bytes = static_cast<double>(g_num_sms) * BK * (bn + BM) * 2.0;
  int want = 1;
  double best = 1e30;
  const int max_s = num_kb / 2 > 32 ? 32 : num_kb / 2;
  for (int sp = 1; sp <= (max_s < 1 ? 1 : max_s); ++sp) {
    const int kb_per = (num_kb + sp - 1) / sp;
    if ((num_kb + kb_per - 1) / kb_per != sp) continue;
    if (workspace_elems / per_split < sp) break;
    const int waves = (tiles * sp + g_num_sms - 1) / g_num_sms;
    // the consumer reads every partial once; no separate reduction pass writes and re-reads them
    const double cost = waves * (kb_per + 2.0) + sp * per_split * 8.0 / block_bytes;
    if (cost < best - 1e-9) { best = cost; want = sp; }
  }
  const int kb_per = (num_kb + want - 1) / want;
  const int k_splits = (num_kb + kb_per - 1) / kb_per;
  *k_splits_out = k_splits;
  CUtensorMap ta, tb;
  const int a_rows = a_box_rows(M, 0);
  int rc = make_tmap_bf16_2d(&ta, A, K, M, lda, BK, a_rows);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tb, B, K, N, ldb, BK, bn);
  if (rc) return rc - 100;
  switch (bn) {
    case 256: return launch_gemm<256, EPI_F32, false, false>(ta, tb, workspace, M, N, K, N, 0, k_splits, per_split, status, g_num_sms, stream,
                                                             WeightGate{nullptr, 0, 0u, 0ull}, pdl_enabled(), a_rows);
    case 128: return launch_gemm<128, EPI_F32, false, false>(ta, tb, workspace, M, N, K, N, 0, k_splits, per_split, status, g_num_sms, stream,
                                                             WeightGate{nullptr, 0, 0u, 0ull}, pdl_enabled(), a_rows);
    case 64: return launch_gemm<64, EPI_F32, false, false>(ta, tb, workspace, M, N, K, N, 0, k_splits, per_split, status, g_num_sms, stream,
                                                             WeightGate{nullptr, 0, 0u, 0ull}, pdl_enabled(), a_rows);
    default: return launch_gemm<32, EPI_F32, false, false>(ta, tb, workspace, M, N, K, N, 0, k_splits, per_split, status, g_num_sms, stream,
                                                             WeightGate{nullptr, 0, 0u, 0ull}, pdl_enabled(), a_rows);
  }
}
