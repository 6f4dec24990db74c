// Column-parallel linear layer with a sequence-parallel input in ONE kernel: all-gather of the activation
// rows over NVLink and the tcgen05 GEMM that consumes them, overlapped block by block.
//
//   every rank holds its own rows of x inside a symmetric buffer X [M, K] (rows of rank q at q * M / world)
//   rank r computes y_r [M, N_r] = X w_r^T with its slice w_r [N_r, K] of the output features
//
// Inside the kernel (persistent, one CTA per SM, 320 threads):
//   warps 6-9  push this rank's own row blocks through the peer pointers into every peer's copy of X, 16-row
//              chunks spread over all CTAs, nearest consumer first, and count each finished part of a chunk
//              in the CONSUMER's ready[row block] (system-scope release). Stores to peer memory are posted and
//              reach link speed; loads from peer memory measured an order of magnitude slower here.
//   warp 0     TMA producer: before the first tile of a row block that came from a peer it waits (bounded)
//              until all chunks of that block have landed, then loads A tiles from the LOCAL X, so every
//              remote byte crosses NVLink exactly once and the tensor cores read local memory
//   warp 1     tcgen05.mma into double-buffered TMEM accumulators
//   warps 2-5  epilogue: TMEM -> bf16 -> y
// Tiles are ordered so that this rank's own rows come first; the peers' rows arrive under those MMAs.
// The copy warps never wait, so every rank's pushes complete and the producers' waits end; all waits are bounded.
// The caller orders calls with a cross-rank barrier (nobody still reads the buffer that is about to be overwritten).
//
// The reference gets this through Megatron's ColumnParallelLinear with sequence parallelism: an NCCL
// all-gather followed by a cuBLAS GEMM (RPEG/runtime/workers/megatron_worker.py:124-303, 676-715).
#include "common.cuh"
#include "rpeg_kernels.h"

#ifdef RPEG_DEV_PROBES
#define RPEG_PROBE(bit) ((probe & (bit)) != 0)
#else
#define RPEG_PROBE(bit) false
#endif

namespace rpeg {

int make_tmap_bf16_2d(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer);

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int THREADS = 320;
constexpr int COPY_THREADS = 128;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int STAGES = 4;
constexpr int TMEM_COLS = 2 * BN;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 512;
constexpr int CHUNK_ROWS = 16;
constexpr int CHUNKS_PER_BLOCK = BM / CHUNK_ROWS;
constexpr unsigned long long READY_WAIT_NS = 10ull * 1000 * 1000 * 1000;

struct Peers {
  void* p[RPEG_MAX_PEERS];
};

__global__ void __launch_bounds__(THREADS, 1)
ag_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, Peers xs,
               Peers readys, __nv_bfloat16* __restrict__ Y, int M, int N, int K, int ldx, int ldy, int rank,
               int world, unsigned epoch, int* status, int probe) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* bar_area = smem + STAGES * STAGE_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(bar_area);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = M / BM;                      // host guarantees M % (BM * world) == 0
  const int n_tiles = (N + BN - 1) / BN;
  const int num_tiles = RPEG_PROBE(4) ? 0 : m_tiles * n_tiles;
  const int num_kb = (K + BK - 1) / BK;
  const int blocks_per_rank = m_tiles / world;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tfull_bar[b], 1); mbar_init(&tempty_bar[b], 4); }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&tmap_a); tma_prefetch_desc(&tmap_b); }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  // Tile order: the owner of the rows advances rank, rank+1, ...; inside an owner's segment groups of 8
  // row blocks sweep N together (A rows stay in L2).
  auto tile_coords = [&](int t, int& tm, int& tn) {
    constexpr int GROUP_M = 8;
    const int seg = blocks_per_rank * n_tiles;
    const int owner_step = t / seg;
    const int r = t - owner_step * seg;
    const int owner = (rank + owner_step) % world;
    const int per_group = GROUP_M * n_tiles;
    const int g = r / per_group;
    const int first_m = g * GROUP_M;
    const int gsize = min(blocks_per_rank - first_m, GROUP_M);
    const int rr = r - g * per_group;
    tm = owner * blocks_per_rank + first_m + (rr % gsize);
    tn = rr / gsize;
  };

  if (warp == 0) {
    if (lane == 0) {
      int stg = 0;
      uint32_t phase = 0;
      int last_ready_block = -1;
      const unsigned expect = epoch * static_cast<unsigned>(CHUNKS_PER_BLOCK * (COPY_THREADS / 32));
      const unsigned* ready = static_cast<const unsigned*>(readys.p[rank]);
      for (int w = blockIdx.x; w < num_tiles; w += gridDim.x) {
        int tm, tn;
        tile_coords(w, tm, tn);
        if (tm / blocks_per_rank != rank && tm != last_ready_block) {
          // rows of a peer: wait until that peer's copy warps have pushed the whole block into this GPU's X
          unsigned seen = 0;
          const uint64_t t0 = global_timer_ns();
          for (;;) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(ready + tm) : "memory");
            if (static_cast<int>(seen - expect) >= 0) break;
            if (*abort_flag) goto producer_done;
            if (global_timer_ns() - t0 > READY_WAIT_NS) {
              record_error(status, RPEG_ERR_FLAG_TIMEOUT, 800, tm);
              *abort_flag = 1;
              goto producer_done;
            }
            __nanosleep(200);
          }
          // the rows were written with ordinary stores; the loads below go through the async proxy
          asm volatile("fence.proxy.async.global;" ::: "memory");
          last_ready_block = tm;
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stg], phase ^ 1u, abort_flag, status, 801)) goto producer_done;
          uint8_t* sa = smem + stg * STAGE_BYTES;
          mbar_expect_tx(&full_bar[stg], STAGE_BYTES);
          tma_load_2d(sa, &tmap_a, &full_bar[stg], kb * BK, tm * BM);
          tma_load_2d(sa + A_BYTES, &tmap_b, &full_bar[stg], kb * BK, tn * BN);
          if (++stg == STAGES) { stg = 0; phase ^= 1u; }
        }
      }
    producer_done:;
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, 0, 0);
      int stg = 0, buf = 0;
      uint32_t phase = 0, acc_phase = 0;
      for (int w = blockIdx.x; w < num_tiles; w += gridDim.x) {
        if (!mbar_wait(&tempty_bar[buf], acc_phase ^ 1u, abort_flag, status, 810)) goto mma_done;
        tc_fence_after_sync();
        const uint32_t tacc = tmem_base + static_cast<uint32_t>(buf * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stg], phase, abort_flag, status, 811)) goto mma_done;
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stg * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_bf16_ss(tacc, make_smem_desc_sw128(sa + k * 32, 16, 1024), make_smem_desc_sw128(sb + k * 32, 16, 1024), idesc,
                         (kb > 0 || k != 0) ? 1u : 0u);
          umma_commit(&empty_bar[stg]);
          if (++stg == STAGES) { stg = 0; phase ^= 1u; }
        }
        umma_commit(&tfull_bar[buf]);
        if (++buf == 2) { buf = 0; acc_phase ^= 1u; }
      }
    mma_done:;
    }
  } else if (warp < 6) {
    const int quad = warp & 3;
    int buf = 0;
    uint32_t acc_phase = 0;
    for (int w = blockIdx.x; w < num_tiles; w += gridDim.x) {
      int tm, tn;
      tile_coords(w, tm, tn);
      const int row = tm * BM + quad * 32 + lane;
      const int n0 = tn * BN;
      if (!__all_sync(0xffffffffu, mbar_wait(&tfull_bar[buf], acc_phase, abort_flag, status, 820))) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(buf * BN);
      __nv_bfloat16* crow = Y + static_cast<size_t>(row) * ldy + n0;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_wait_ld();
        if (n0 + c * 32 < N) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            if (n0 + c * 32 + v * 8 < N) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]));
              o.y = pack_bf16x2(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
              o.z = pack_bf16x2(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
              o.w = pack_bf16x2(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
              *reinterpret_cast<uint4*>(crow + c * 32 + v * 8) = o;
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[buf]);
      if (++buf == 2) { buf = 0; acc_phase ^= 1u; }
    }
  } else {
    // ---- copy warps: PUSH this rank's own rows into every peer's X (remote stores are posted and run at link
    // speed; remote loads are not), nearest consumer first: rank r - 1 multiplies these rows second, r - 2 third, ...
    const int ct = threadIdx.x - (THREADS - COPY_THREADS);          // 0..127
    const int cw = ct >> 5;                                          // copy warp 0..3
    const __nv_bfloat16* x_local = static_cast<const __nv_bfloat16*>(xs.p[rank]);
    const int vec_per_row = K >> 3;                                  // 16-byte vectors of one row
    const int chunk_vecs = CHUNK_ROWS * vec_per_row;
    const int per_peer = blocks_per_rank * CHUNKS_PER_BLOCK;
    const int push_chunks = (world - 1) * per_peer;
    for (int g = blockIdx.x; g < push_chunks && !RPEG_PROBE(1); g += gridDim.x) {
      const int step = g / per_peer, rest = g - step * per_peer;
      const int dst_rank = (rank - 1 - step + 2 * world) % world;
      const int blk = rank * blocks_per_rank + rest / CHUNKS_PER_BLOCK;
      const int row0 = blk * BM + (rest % CHUNKS_PER_BLOCK) * CHUNK_ROWS;
      __nv_bfloat16* x_peer = static_cast<__nv_bfloat16*>(xs.p[dst_rank]);
      constexpr int UNROLL = 8;
      for (int i0 = ct; i0 < chunk_vecs; i0 += COPY_THREADS * UNROLL) {
        uint4 v[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const int i = i0 + u * COPY_THREADS;
          if (i < chunk_vecs)
            v[u] = *reinterpret_cast<const uint4*>(x_local + static_cast<size_t>(row0 + i / vec_per_row) * ldx + (i % vec_per_row) * 8);
        }
        if (RPEG_PROBE(2)) continue;
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const int i = i0 + u * COPY_THREADS;
          if (i < chunk_vecs)
            *reinterpret_cast<uint4*>(x_peer + static_cast<size_t>(row0 + i / vec_per_row) * ldx + (i % vec_per_row) * 8) = v[u];
        }
      }
      // this warp's part of the chunk is on its way: make it visible system-wide, then count it at the consumer
      __threadfence_system();
      __syncwarp();
      if ((ct & 31) == 0) {
        unsigned* ctr = static_cast<unsigned*>(readys.p[dst_rank]) + blk;
        asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(ctr) : "memory");
      }
      (void)cw;
    }
  }

  __syncwarp();
  if (*abort_flag) __nanosleep(200000);
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace
}  // namespace rpeg

using namespace rpeg;

// Timing probes exist only in builds with -DRPEG_DEV_PROBES (bit 0 skips the pulls, bit 1 drops the local stores, bit 2
// skips the GEMM tiles; results are wrong with any bit set).
#ifdef RPEG_DEV_PROBES
static int g_ag_probe = 0;
extern "C" void rpeg_ag_gemm_set_probe(int bits) { g_ag_probe = bits; }
#else
static constexpr int g_ag_probe = 0;
#endif

// xs[q]: rank q's X buffer ([M, ldx] bf16, symmetric); on entry rank q's own rows are valid in xs[q]. W [N, ldw]
// bf16 local; Y [M, ldy] bf16 local. readys[q]: rank q's arrival counters uint32[M / 128] (symmetric, zeroed once);
// `epoch` counts calls from 1. M must be a multiple of 128 * world; N, K, ld* multiples of 8.
extern "C" int rpeg_ag_gemm(void* const* xs, const void* W, void* Y, void* const* readys, int M, int N, int K, int ldx, int ldw,
                            int ldy, int rank, int world, unsigned epoch, int* status, void* stream_v) {
  if (world < 1 || world > RPEG_MAX_PEERS || rank < 0 || rank >= world) return -2;
  if (M <= 0 || N <= 0 || K <= 0 || (M % (BM * world)) != 0 || (N & 7) || (K & 7) || (ldx & 7) || (ldw & 7) || (ldy & 7)) return -3;
  static int num_sms = 0;
  static bool configured = false;
  if (num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  if (!configured) {
    if (cudaFuncSetAttribute(ag_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) return -20;
    configured = true;
  }
  CUtensorMap ta, tb;
  int rc = make_tmap_bf16_2d(&ta, xs[rank], K, M, ldx, BK, BM);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tb, W, K, N, ldw, BK, BN);
  if (rc) return rc - 100;
  Peers px, pr;
  for (int i = 0; i < RPEG_MAX_PEERS; ++i) {
    px.p[i] = i < world ? xs[i] : nullptr;
    pr.p[i] = i < world ? readys[i] : nullptr;
  }
  const int tiles = (M / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < num_sms ? tiles : num_sms;
  ag_gemm_kernel<<<grid, THREADS, SMEM_BYTES, static_cast<cudaStream_t>(stream_v)>>>(ta, tb, px, pr, static_cast<__nv_bfloat16*>(Y), M, N,
                                                                                   K, ldx, ldy, rank, world, epoch, status, g_ag_probe);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}
