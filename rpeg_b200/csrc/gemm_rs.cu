// Row-parallel linear layer across tensor-parallel ranks in ONE kernel: tcgen05 GEMM whose epilogue
// pushes its partial tile over NVLink to the rank that owns those rows, followed (same launch) by the
// owner's reduction of the partials it received.
//
//   rank r holds x_r [M, K_r] and w_r [N, K_r] (its slice of the contraction dimension)
//   partial_r = x_r w_r^T                                     tcgen05.mma, fp32 in TMEM
//   y[rows of rank q] = sum_r partial_r[rows of rank q]       reduce-scatter over rows, bf16 out
//   (all_gather = 1: the owner also stores the reduced rows into every peer's y => all-reduce)
//
// Phase 1 (persistent tile loop, identical pipeline to gemm.cu): the epilogue converts a 128 x BN
// accumulator to bf16 and stores it into the owner's staging buffer stage_q[r][local_row][col]
// (plain 16-byte stores to peer memory; the local rank's own partial goes to local memory). When the
// an epilogue warp is done with its 32 rows of a tile, it makes the stores visible system-wide and adds 1
// to the owner's arrival counter of that 128-row block. Transfers of tile i overlap the MMAs of tile
// i+1 because the accumulator is double buffered in TMEM.
// Phase 2: all CTAs take 16-row items of the rows this rank owns, wait (bounded) until the block's counter
// reached epoch * n_tiles * world * 4 (one arrival per epilogue warp), stream the `world` partials through shared
// memory with bulk copies, sum them in fp32 and write bf16.
// No CTA waits on a peer before it has issued all of its own pushes, so the ranks cannot deadlock;
// every wait is bounded by %globaltimer and reports through the status word.
//
// The reference reaches this pattern through Megatron's RowParallelLinear: a cuBLAS GEMM followed by
// an NCCL reduce-scatter / all-reduce (RPEG/runtime/workers/megatron_worker.py:676-715 builds the
// model; tensor-parallel groups are made in :124-303).
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
constexpr int THREADS = 192;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int STAGES = 4;
constexpr int TMEM_COLS = 2 * BN;
constexpr int EPI_ROW_BYTES = 128 + 16;            // 64 bf16 per row, padded so 16-byte accesses spread over the banks
constexpr int EPI_WARP_BYTES = 32 * EPI_ROW_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 512 + 4 * EPI_WARP_BYTES;
constexpr unsigned long long PEER_WAIT_NS = 10ull * 1000 * 1000 * 1000;

struct Peers {
  void* p[RPEG_MAX_PEERS];
};

__global__ void __launch_bounds__(THREADS, 1)
gemm_rs_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, Peers stage,
               Peers counters, Peers outs, int M, int N, int K, int ldo, int rank, int world, unsigned epoch,
               int all_gather, int probe, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* bar_area = smem + STAGES * STAGE_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(bar_area);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* epi_area = bar_area + 512;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = M / BM;                       // host guarantees M % (BM * world) == 0
  const int n_tiles = (N + BN - 1) / BN;
  const int num_tiles = m_tiles * n_tiles;
  const int num_kb = (K + BK - 1) / BK;
  const int blocks_per_rank = m_tiles / world;      // 128-row blocks owned by one rank
  const int rows_per_rank = blocks_per_rank * BM;

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

  // Tile order: start with the row blocks of the NEXT rank and end with this rank's own, so remote
  // owners receive their partials early and the local partial (no NVLink) comes last.
  // Inside an owner's segment, groups of 8 row blocks sweep N together so the A rows stay in L2.
  auto tile_coords = [&](int t, int& tm, int& tn) {
    constexpr int GROUP_M = 8;
    const int seg = blocks_per_rank * n_tiles;
    const int owner_step = t / seg;
    const int r = t - owner_step * seg;
    const int owner = (rank + 1 + owner_step) % world;
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
      for (int w = blockIdx.x; w < num_tiles; w += gridDim.x) {
        int tm, tn;
        tile_coords(w, tm, tn);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stg], phase ^ 1u, abort_flag, status, 700)) goto producer_done;
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
        if (!mbar_wait(&tempty_bar[buf], acc_phase ^ 1u, abort_flag, status, 710)) goto mma_done;
        tc_fence_after_sync();
        const uint32_t tacc = tmem_base + static_cast<uint32_t>(buf * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stg], phase, abort_flag, status, 711)) goto mma_done;
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
  } else {
    const int quad = warp & 3;
    int buf = 0;
    uint32_t acc_phase = 0;
    for (int w = blockIdx.x; w < num_tiles; w += gridDim.x) {
      int tm, tn;
      tile_coords(w, tm, tn);
      const int owner = tm / blocks_per_rank;
      const int n0 = tn * BN;
      if (!__all_sync(0xffffffffu, mbar_wait(&tfull_bar[buf], acc_phase, abort_flag, status, 720))) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(buf * BN);
      // owner's staging: [world][rows_per_rank][N] bf16; this rank writes slab `rank`. The accumulator is
      // read one row per lane, so it goes through a small per-warp shared buffer and leaves as whole
      // 128-byte row segments (4 rows per store instruction): NVLink moves full-size packets instead of
      // one 16-byte fragment per lane.
      __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(stage.p[owner]) +
                           (static_cast<size_t>(rank) * rows_per_rank + (tm - owner * blocks_per_rank) * BM + quad * 32) * N + n0;
      uint8_t* my_epi = epi_area + quad * EPI_WARP_BYTES;
#pragma unroll 1
      for (int c = 0; c < BN / 64; ++c) {
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 64 + hh * 32, r);
          tmem_wait_ld();
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]));
            o.y = pack_bf16x2(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
            o.z = pack_bf16x2(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
            o.w = pack_bf16x2(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
            *reinterpret_cast<uint4*>(my_epi + lane * EPI_ROW_BYTES + hh * 64 + v * 16) = o;
          }
        }
        __syncwarp();
        const int col_base = n0 + c * 64;
        if (col_base < N) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int rr = 4 * j + (lane >> 3), ch = lane & 7;
            const uint4 v = *reinterpret_cast<const uint4*>(my_epi + rr * EPI_ROW_BYTES + ch * 16);
            if (col_base + ch * 8 < N) *reinterpret_cast<uint4*>(dst + static_cast<size_t>(rr) * N + c * 64 + ch * 8) = v;
          }
        }
        __syncwarp();
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[buf]);
      // this warp's 32 rows of the tile are stored: publish them to the owner (4 arrivals per tile, one
      // per epilogue warp, so no cross-warp barrier is needed on this path)
      if (!RPEG_PROBE(1)) __threadfence_system();
      __syncwarp();
      if (lane == 0) {
        unsigned* ctr = static_cast<unsigned*>(counters.p[owner]) + (tm - owner * blocks_per_rank);
        asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(ctr) : "memory");
      }
      if (++buf == 2) { buf = 0; acc_phase ^= 1u; }
    }
  }

  // ---- phase 2: reduce the rows this rank owns.
  // A work item is 16 consecutive rows of a 128-row block: one contiguous 32 * N byte region per source rank in
  // the staging buffer. One elected thread streams the `world` regions through the (now idle) operand stages with
  // bulk copies (cp.async.bulk global -> shared, complete_tx on an mbarrier), 8 KiB per source and step and up to
  // 192 KiB in flight per SM, so the tail runs at memory speed with one CTA per SM; five warps add the slots up in
  // fp32 and store bf16. Plain loads from six warps kept too few bytes in flight: measured ~1 TB/s.
  __syncwarp();
  __syncthreads();
  if (*abort_flag) {
    __nanosleep(200000);
  } else if (!RPEG_PROBE(2)) {
    constexpr int SLOT_BYTES = 8192;
    constexpr int MAX_GROUPS = 24;
    constexpr int SUB_ROWS = 16;
    constexpr int CONSUMER_WARPS = THREADS / 32 - 1;
    const int group_bytes = world * SLOT_BYTES;
    const int n_groups = min(MAX_GROUPS, (STAGES * STAGE_BYTES) / group_bytes);
    uint64_t* rfull = reinterpret_cast<uint64_t*>(bar_area + 128);
    uint64_t* rempty = rfull + MAX_GROUPS;
    if (threadIdx.x == 0) {
      for (int g = 0; g < n_groups; ++g) { mbar_init(&rfull[g], 1); mbar_init(&rempty[g], CONSUMER_WARPS); }
      fence_mbar_init();
    }
    __syncthreads();
    const unsigned expect = epoch * static_cast<unsigned>(n_tiles * world * 4);
    const unsigned* my_ctr = static_cast<const unsigned*>(counters.p[rank]);
    const uint8_t* my_stage = static_cast<const uint8_t*>(stage.p[rank]);
    const int items = blocks_per_rank * (BM / SUB_ROWS);
    const long long region_bytes = static_cast<long long>(SUB_ROWS) * N * 2;
    const int steps = static_cast<int>((region_bytes + SLOT_BYTES - 1) / SLOT_BYTES);
    if (warp == 0) {
      if (lane == 0) {
        int g = 0;
        uint32_t ph = 0;
        int waited_blk = -1;
        for (int it = blockIdx.x; it < items; it += gridDim.x) {
          const int blk = it / (BM / SUB_ROWS), sub = it % (BM / SUB_ROWS);
          if (blk != waited_blk) {
            unsigned seen = 0;
            const uint64_t t0 = global_timer_ns();
            for (;;) {
              asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(my_ctr + blk) : "memory");
              if (static_cast<int>(seen - expect) >= 0) break;
              if (*abort_flag) goto reduce_producer_done;
              if (global_timer_ns() - t0 > PEER_WAIT_NS) {
                record_error(status, RPEG_ERR_FLAG_TIMEOUT, 730, blk);
                *abort_flag = 1;
                goto reduce_producer_done;
              }
              __nanosleep(100);
            }
            // the partials were written with ordinary (local and peer) stores; the bulk copies read through the async proxy
            asm volatile("fence.proxy.async.global;" ::: "memory");
            waited_blk = blk;
          }
          const size_t row_off = (static_cast<size_t>(blk) * BM + sub * SUB_ROWS) * N * 2;
          for (int c = 0; c < steps; ++c) {
            if (!mbar_wait(&rempty[g], ph ^ 1u, abort_flag, status, 731)) goto reduce_producer_done;
            const long long off = static_cast<long long>(c) * SLOT_BYTES;
            const uint32_t bytes = static_cast<uint32_t>(min(static_cast<long long>(SLOT_BYTES), region_bytes - off));
            mbar_expect_tx(&rfull[g], bytes * world);
            for (int sr = 0; sr < world; ++sr) {
              const uint8_t* src = my_stage + static_cast<size_t>(sr) * rows_per_rank * N * 2 + row_off + off;
              asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                               smem_u32(smem + g * group_bytes + sr * SLOT_BYTES)),
                           "l"(src), "r"(bytes), "r"(smem_u32(&rfull[g]))
                           : "memory");
            }
            if (++g == n_groups) { g = 0; ph ^= 1u; }
          }
        }
      reduce_producer_done:;
      }
    } else {
      const int ctid = threadIdx.x - 32;
      constexpr int CONSUMERS = CONSUMER_WARPS * 32;
      int g = 0;
      uint32_t ph = 0;
      bool alive = true;
      for (int it = blockIdx.x; it < items && alive; it += gridDim.x) {
        const int blk = it / (BM / SUB_ROWS), sub = it % (BM / SUB_ROWS);
        const int row_base = blk * BM + sub * SUB_ROWS;
        for (int c = 0; c < steps; ++c) {
          if (!__all_sync(0xffffffffu, mbar_wait(&rfull[g], ph, abort_flag, status, 732))) { alive = false; break; }
          const long long off = static_cast<long long>(c) * SLOT_BYTES;
          const int nvec = static_cast<int>(min(static_cast<long long>(SLOT_BYTES), region_bytes - off) >> 4);
          const uint8_t* slot0 = smem + g * group_bytes;
          for (int v = ctid; v < nvec; v += CONSUMERS) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int sr = 0; sr < world; ++sr) {
              const uint4 x = *reinterpret_cast<const uint4*>(slot0 + sr * SLOT_BYTES + v * 16);
              const float2 a = unpack_bf16x2(x.x), b2 = unpack_bf16x2(x.y), c2 = unpack_bf16x2(x.z), d2 = unpack_bf16x2(x.w);
              acc[0] += a.x; acc[1] += a.y; acc[2] += b2.x; acc[3] += b2.y;
              acc[4] += c2.x; acc[5] += c2.y; acc[6] += d2.x; acc[7] += d2.y;
            }
            const long long e = (off >> 1) + static_cast<long long>(v) * 8;      // element inside the 16-row region
            const int row = row_base + static_cast<int>(e / N), col = static_cast<int>(e % N);
            uint4 o;
            o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
            o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
            if (all_gather) {
              const size_t o_off = (static_cast<size_t>(rank) * rows_per_rank + row) * ldo + col;
              for (int q = 0; q < world; ++q) *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(outs.p[q]) + o_off) = o;
            } else {
              *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(outs.p[rank]) + static_cast<size_t>(row) * ldo + col) = o;
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&rempty[g]);
          if (++g == n_groups) { g = 0; ph ^= 1u; }
        }
      }
    }
    __syncwarp();
    if (*abort_flag) __nanosleep(200000);        // bulk copies that were in flight when a wait gave up
  }
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

// Timing probes exist only in builds with -DRPEG_DEV_PROBES (bit 0 drops the system fence before the arrival counter,
// bit 1 skips the owner's reduction; results are wrong with either bit set). The product build has neither the
// switch nor the branches.
#ifdef RPEG_DEV_PROBES
static int g_probe = 0;
extern "C" void rpeg_gemm_rs_set_probe(int bits) { g_probe = bits; }
#else
static constexpr int g_probe = 0;
#endif

// A [M, K] (lda), B [N, K] (ldb), both K-major bf16 in this rank's memory. stage[q]: rank q's staging
// buffer of world * (M / world) * N bf16; counters[q]: rank q's M / world / 128 arrival counters
// (uint32, zeroed once; `epoch` counts calls from 1); outs[q]: rank q's output: [M / world, ldo]
// (reduce-scatter) or [M, ldo] (all_gather = 1). M must be a multiple of 128 * world, N of 8.
extern "C" int rpeg_gemm_rs(const void* A, const void* B, int M, int N, int K, int lda, int ldb, void* const* stage,
                            void* const* counters, void* const* outs, int ldo, int rank, int world, unsigned epoch,
                            int all_gather, int* status, void* stream_v) {
  if (world < 1 || world > RPEG_MAX_PEERS || rank < 0 || rank >= world) return -2;
  if (M <= 0 || N <= 0 || K <= 0 || (M % (BM * world)) != 0 || (N & 7) || (K & 7) || (lda & 7) || (ldb & 7) || (ldo & 7)) return -3;
  static int num_sms = 0;
  static bool configured = false;
  if (num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_rs_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) return -20;
    configured = true;
  }
  CUtensorMap ta, tb;
  int rc = make_tmap_bf16_2d(&ta, A, K, M, lda, BK, BM);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tb, B, K, N, ldb, BK, BN);
  if (rc) return rc - 100;
  Peers ps, pc, po;
  for (int i = 0; i < RPEG_MAX_PEERS; ++i) {
    ps.p[i] = i < world ? stage[i] : nullptr;
    pc.p[i] = i < world ? counters[i] : nullptr;
    po.p[i] = i < world ? outs[i] : nullptr;
  }
  const int tiles = (M / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < num_sms ? tiles : num_sms;
  gemm_rs_kernel<<<grid, THREADS, SMEM_BYTES, static_cast<cudaStream_t>(stream_v)>>>(ta, tb, ps, pc, po, M, N, K, ldo, rank, world,
                                                                                   epoch, all_gather, g_probe, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}
