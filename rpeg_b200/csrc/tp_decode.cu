// Collectives of the tensor-parallel decode step for sm_100a, fused with the work that follows them.
//
// In tensor-parallel decoding every GPU holds 1/world of each weight matrix and of the KV heads and works on ALL
// rows of the batch. The attention output projection and the MLP down projection leave a partial sum [B, d] on
// every rank; what the next layer needs is RMSNorm(sum over ranks + residual), identical on every rank.
//
//   tp_allreduce_rmsnorm : rank r owns the rows [r*B/world, (r+1)*B/world). One kernel
//                             waits until every rank's partial is complete            (flag exchange, bounded)
//                             reduces its rows over all ranks                         multimem.ld_reduce (NVSwitch adds
//                                                                                     in fp32), or loads from each peer
//                             adds the residual, rounds to bf16 = new residual stream, normalises
//                             stores both results into EVERY rank's buffers           multimem.st, or a store per peer
//                             tells the peers, and leaves only when all peers told it (flag exchange, bounded)
//                          i.e. reduce-scatter, residual add, RMSNorm and all-gather of a row-parallel linear's
//                          output in one launch; when it returns on a rank, that rank's buffers are complete.
//   tp_allreduce_rmsnorm_ll : the same result for FEW rows (the long tail of a generation, where the step is bound by
//                          latency, not by bytes). One exchange instead of three: every rank pushes its partial rows
//                          into a slot of its own in EVERY region as 8-byte units {two bf16 values, call number}, the
//                          receivers poll the units themselves (no flag after the data, hence no fence that waits for
//                          the stores to be acknowledged), and every rank sums the slots of all ranks in rank order,
//                          so the results are the same bits everywhere. Twice the bytes, about a third of the latency.
//   tp_allgather_cols    : vocabulary-parallel LM head: every rank wrote logits[:, r*Vloc .. (r+1)*Vloc) into its
//                          own copy of the [B, V] buffer; the kernel pushes that block into all peers' copies and
//                          waits until the peers' blocks have landed here.
//
// All buffers live at the same offset of one symmetric region per rank (`TpComm::peer`), optionally mapped on an
// NVLink multicast address (`TpComm::mc`). Flags are monotonically increasing call numbers kept on the device
// (`state[0]`), so the kernels replay unchanged inside a CUDA graph. Every spin is bounded; a wait that runs out
// records RPEG_ERR_FLAG_TIMEOUT in the status word. From then on every launch of these kernels on this GPU returns
// at once, without waiting and without touching peer or multicast memory (a peer that stopped answering may be
// gone), until the host has read and cleared the status word: a lost rank costs one timeout, not one per launch.
//
// Reference behaviour replaced: the tensor-parallel all-reduces megatron-core issues inside
// linear_proj / linear_fc2 during generation (RPEG/runtime/workers/megatron_worker.py:2301-3107, static-KV
// forward at :2782; priced in RPEG/model/cost.py:330-405,538-654) and the logits all-gather of
// runtime_gather_output=True (megatron_worker.py:2078).
#include "common.cuh"
#include "rpeg_kernels.h"

namespace rpeg {

struct TpComm {
  void* peer[RPEG_MAX_PEERS];  // base of every rank's region (own included), rank order
  void* mc;                    // multicast address of the region, or nullptr: plain peer loads / stores
  int rank;
  int world;
};

__device__ __forceinline__ void mc_ld_reduce_bf16x8(const void* mc_addr, uint32_t (&v)[4]) {
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3])
               : "l"(mc_addr)
               : "memory");
}
__device__ __forceinline__ void mc_st_16(void* mc_addr, const uint32_t (&v)[4]) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v[0]), "r"(v[1]),
               "r"(v[2]), "r"(v[3])
               : "memory");
}
__device__ __forceinline__ void peer_ld_16(const void* addr, uint32_t (&v)[4]) {
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3])
               : "l"(addr)
               : "memory");
}
__device__ __forceinline__ void peer_st_16(void* addr, const uint32_t (&v)[4]) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "r"(v[0]), "r"(v[1]), "r"(v[2]),
               "r"(v[3])
               : "memory");
}

// Thread t < world: tell rank t that this rank reached `epoch` (word `rank` of its flag array), then wait until
// rank t told this rank the same. Returns false when the wait ran out.
__device__ __forceinline__ bool exchange_flags(const TpComm& c, long long flag_off, unsigned epoch,
                                               unsigned long long timeout_ns, int* status, int where) {
  const int t = threadIdx.x;
  if (t >= c.world) return true;
  unsigned* theirs = reinterpret_cast<unsigned*>(static_cast<char*>(c.peer[t]) + flag_off) + c.rank;
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
  const unsigned* mine = reinterpret_cast<const unsigned*>(static_cast<const char*>(c.peer[c.rank]) + flag_off) + t;
  const uint64_t t0 = global_timer_ns();
  for (;;) {
    unsigned seen;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
    if (static_cast<int>(seen - epoch) >= 0) return true;
    if (global_timer_ns() - t0 > timeout_ns) {
      record_error(status, RPEG_ERR_FLAG_TIMEOUT, where, t);
      return false;
    }
    __nanosleep(32);
  }
}

// Region layout (byte offsets, the same on every rank): part [B, d] bf16 partial sums, y [B, d] bf16 normalised
// output, h [B, d] bf16 residual stream (h_off < 0: not wanted), flags: two arrays of RPEG_MAX_PEERS uint32
// ("partials ready", "outputs landed"). `res` is this rank's copy of the residual stream (may alias the h buffer:
// a rank reads and writes only its own rows of it). state[0] = calls finished so far, state[1] = blocks finished.
template <int NV, bool MC>
__global__ void __launch_bounds__(256)
tp_allreduce_rmsnorm_kernel(TpComm c, long long part_off, const __nv_bfloat16* __restrict__ res,
                            const __nv_bfloat16* __restrict__ w, long long y_off, long long h_off, int B, int d, float eps,
                            long long flag_off, unsigned* __restrict__ state, unsigned long long timeout_ns, int* status) {
  __shared__ float warp_ss[8];
  // Launched as a programmatic dependent: the next kernel of the step (a GEMM) may become resident now and fetch its
  // first weight tiles while this kernel talks to the peers; this kernel itself waits for its producer (the GEMM that
  // wrote the partial sums) before it reads or signals anything.
  griddep_launch();
  griddep_wait();
  if (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) return;   // an earlier wait ran out: stand down
  const unsigned epoch = state[0] + 1u;
  const int rows_per = (B + c.world - 1) / c.world;
  const int row = c.rank * rows_per + static_cast<int>(blockIdx.x);
  const bool has_row = static_cast<int>(blockIdx.x) < rows_per && row < B;
  // every block needs the peers' partials, so every block waits; only block 0 announces this rank
  __shared__ int gave_up;
  if (threadIdx.x == 0) gave_up = 0;
  __syncthreads();
  if (blockIdx.x == 0) {
    if (!exchange_flags(c, flag_off, epoch, timeout_ns, status, 700)) gave_up = 1;
  } else if (threadIdx.x < c.world) {
    const unsigned* mine = reinterpret_cast<const unsigned*>(static_cast<const char*>(c.peer[c.rank]) + flag_off) + threadIdx.x;
    const uint64_t t0 = global_timer_ns();
    for (;;) {
      unsigned seen;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
      if (static_cast<int>(seen - epoch) >= 0) break;
      if (global_timer_ns() - t0 > timeout_ns) { record_error(status, RPEG_ERR_FLAG_TIMEOUT, 701, threadIdx.x); gave_up = 1; break; }
      __nanosleep(32);
    }
  }
  __syncthreads();
  if (gave_up) return;   // a peer did not answer: do not read or write its memory

  const int nvec = d >> 3;
  float v[NV][8];
  float ss = 0.f;
  if (has_row) {
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int i = threadIdx.x + k * 256;
      if (i < nvec) {
        const long long off = part_off + (static_cast<long long>(row) * d + i * 8) * 2;
        uint32_t a[4];
        if constexpr (MC) {
          mc_ld_reduce_bf16x8(static_cast<const char*>(c.mc) + off, a);
#pragma unroll
          for (int e = 0; e < 4; ++e) { const float2 f = unpack_bf16x2(a[e]); v[k][2 * e] = f.x; v[k][2 * e + 1] = f.y; }
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) v[k][e] = 0.f;
          for (int p = 0; p < c.world; ++p) {
            peer_ld_16(static_cast<const char*>(c.peer[p]) + off, a);
#pragma unroll
            for (int e = 0; e < 4; ++e) { const float2 f = unpack_bf16x2(a[e]); v[k][2 * e] += f.x; v[k][2 * e + 1] += f.y; }
          }
        }
        if (res != nullptr) {
          const uint4 r = reinterpret_cast<const uint4*>(res + static_cast<size_t>(row) * d)[i];
          const uint32_t* pr = reinterpret_cast<const uint32_t*>(&r);
#pragma unroll
          for (int e = 0; e < 4; ++e) { const float2 f = unpack_bf16x2(pr[e]); v[k][2 * e] += f.x; v[k][2 * e + 1] += f.y; }
        }
        // the residual stream is kept in bf16: round here so the norm sees exactly what is stored
        uint32_t hv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          hv[e] = pack_bf16x2(v[k][2 * e], v[k][2 * e + 1]);
          const float2 f = unpack_bf16x2(hv[e]);
          v[k][2 * e] = f.x; v[k][2 * e + 1] = f.y;
          ss += f.x * f.x + f.y * f.y;
        }
        if (h_off >= 0) {
          const long long o = h_off + (static_cast<long long>(row) * d + i * 8) * 2;
          if constexpr (MC) {
            mc_st_16(static_cast<char*>(c.mc) + o, hv);
          } else {
            for (int p = 0; p < c.world; ++p) peer_st_16(static_cast<char*>(c.peer[p]) + o, hv);
          }
        }
      }
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) warp_ss[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (has_row) {
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
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 b = unpack_bf16x2(pw[e]);
          o[e] = pack_bf16x2(v[k][2 * e] * rstd * b.x, v[k][2 * e + 1] * rstd * b.y);
        }
        const long long off = y_off + (static_cast<long long>(row) * d + i * 8) * 2;
        if constexpr (MC) {
          mc_st_16(static_cast<char*>(c.mc) + off, o);
        } else {
          for (int p = 0; p < c.world; ++p) peer_st_16(static_cast<char*>(c.peer[p]) + off, o);
        }
      }
    }
  }
  // this block's stores are on their way; the last block of the rank tells the peers and waits for theirs
  __threadfence_system();
  __syncthreads();
  __shared__ unsigned last;
  if (threadIdx.x == 0) last = (atomicAdd(&state[1], 1u) == gridDim.x - 1u) ? 1u : 0u;
  __syncthreads();
  if (last) {
    exchange_flags(c, flag_off + RPEG_MAX_PEERS * 4, epoch, timeout_ns, status, 702);
    __syncthreads();
    if (threadIdx.x == 0) {
      state[1] = 0u;
      state[0] = epoch;
    }
  }
}

// One-shot variant for few rows. Slot layout inside the region, from `ll_off`: [2 parities][world senders][ll_rows]
// rows of d / 2 units, a unit being {bf16x2 data, uint32 call number}. Block b owns row b on both sides: it pushes
// this rank's partial of the row to all ranks and reduces the row from all ranks' slots. state[2] counts these
// calls; the parity of the call number selects the slot set, which is enough because a rank can be at most one call
// ahead of a peer (it cannot finish call k + 1 before that peer has sent its part of k + 1, i.e. has finished call k).
__device__ unsigned long long g_tp_trace[4];   // %globaltimer at entry / after the push / when all slots were complete
__device__ int g_tp_trace_on;

constexpr int LL_THREADS = 1024;   // one 16-byte store per thread for d = 4096: the whole row is in flight at once

template <int NP, bool MC>
__global__ void __launch_bounds__(LL_THREADS)
tp_allreduce_rmsnorm_ll_kernel(TpComm c, long long part_off, const float* __restrict__ parts, int splits, long long split_stride,
                               const __nv_bfloat16* __restrict__ res, const __nv_bfloat16* __restrict__ w, long long y_off,
                               long long h_off, int B, int d, float eps, long long ll_off, int ll_rows,
                               unsigned* __restrict__ state, unsigned long long timeout_ns, int* status) {
  __shared__ float warp_ss[LL_THREADS / 32];
  griddep_launch();
  griddep_wait();
  // the three words this launch depends on are fetched together (one memory round trip, not three in a row)
  const int poisoned = status != nullptr ? *reinterpret_cast<volatile int*>(status) : 0;
  const unsigned calls = *reinterpret_cast<volatile unsigned*>(state + 2);
  const int trace_on = *reinterpret_cast<volatile int*>(&g_tp_trace_on);
  if (poisoned != 0) return;   // an earlier wait ran out: stand down
  const bool trace = trace_on != 0 && blockIdx.x == 0 && threadIdx.x == 0;
  if (trace) g_tp_trace[0] = global_timer_ns();
  const unsigned epoch = calls + 1u;
  const int row = static_cast<int>(blockIdx.x);
  const int pairs = d >> 2;                                   // 16-byte stores: two units = four bf16 values
  const long long row_bytes = static_cast<long long>(d) * 4;  // d / 2 units of 8 bytes
  const long long set_off = ll_off + static_cast<long long>(epoch & 1u) * c.world * ll_rows * row_bytes;
  char* own = static_cast<char*>(c.peer[c.rank]);
  // ---- push this rank's partial of the row into its slot in every region
  {
    const uint2* src = reinterpret_cast<const uint2*>(own + part_off + static_cast<long long>(row) * d * 2);
    const long long dst = set_off + (static_cast<long long>(c.rank) * ll_rows + row) * row_bytes;
#pragma unroll
    for (int k = 0; k < NP; ++k) {
      const int i = threadIdx.x + k * LL_THREADS;
      if (i < pairs) {
        uint2 v;
        if (parts != nullptr) {
          // the producer was a split-K GEMM: its fp32 partial slabs are summed here instead of by a kernel of their own
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int sp = 0; sp < splits; ++sp) {
            const float4 q = reinterpret_cast<const float4*>(parts + sp * split_stride + static_cast<long long>(row) * d)[i];
            acc.x += q.x; acc.y += q.y; acc.z += q.z; acc.w += q.w;
          }
          v.x = pack_bf16x2(acc.x, acc.y);
          v.y = pack_bf16x2(acc.z, acc.w);
        } else {
          v = src[i];
        }
        const uint32_t u[4] = {v.x, epoch, v.y, epoch};
        if constexpr (MC) {
          mc_st_16(static_cast<char*>(c.mc) + dst + static_cast<long long>(i) * 16, u);
        } else {
          for (int p = 0; p < c.world; ++p) peer_st_16(static_cast<char*>(c.peer[p]) + dst + static_cast<long long>(i) * 16, u);
        }
      }
    }
  }
  if (trace) g_tp_trace[1] = global_timer_ns();
  // the residual and the norm weights do not depend on the peers: their loads are in flight while the units arrive
  uint2 res_v[NP], w_v[NP];
#pragma unroll
  for (int k = 0; k < NP; ++k) {
    const int i = threadIdx.x + k * LL_THREADS;
    res_v[k] = make_uint2(0u, 0u);
    w_v[k] = make_uint2(0u, 0u);
    if (i < pairs) {
      if (res != nullptr) res_v[k] = reinterpret_cast<const uint2*>(res + static_cast<size_t>(row) * d)[i];
      w_v[k] = reinterpret_cast<const uint2*>(w)[i];
    }
  }
  // ---- collect: the units of every sender validate themselves. All senders' loads of a thread are in flight
  // together; the sum runs in rank order once they are complete (the same bits on every rank).
  float v[NP][4];
  const uint64_t t0 = global_timer_ns();
  const char* slots = own + set_off + static_cast<long long>(row) * row_bytes;
  const long long sender_stride = static_cast<long long>(ll_rows) * row_bytes;
#pragma unroll
  for (int k = 0; k < NP; ++k) {
    const int i = threadIdx.x + k * LL_THREADS;
    v[k][0] = v[k][1] = v[k][2] = v[k][3] = 0.f;
    if (i < pairs) {
      uint32_t a[RPEG_MAX_PEERS][4];
      unsigned pending = (1u << c.world) - 1u, spins = 0;
      while (pending != 0u) {
#pragma unroll
        for (int p = 0; p < RPEG_MAX_PEERS; ++p)
          if ((pending >> p) & 1u) peer_ld_16(slots + p * sender_stride + static_cast<long long>(i) * 16, a[p]);
#pragma unroll
        for (int p = 0; p < RPEG_MAX_PEERS; ++p)
          if (((pending >> p) & 1u) && a[p][1] == epoch && a[p][3] == epoch) pending &= ~(1u << p);
        if (pending != 0u && (++spins & 31u) == 0u && global_timer_ns() - t0 > timeout_ns) {
          record_error(status, RPEG_ERR_FLAG_TIMEOUT, 720, static_cast<int>(pending));
          break;                                               // give up: finish on what is there, the host sees the status
        }
      }
#pragma unroll
      for (int p = 0; p < RPEG_MAX_PEERS; ++p) {
        if (p < c.world) {
          const float2 f0 = unpack_bf16x2(a[p][0]), f1 = unpack_bf16x2(a[p][2]);
          v[k][0] += f0.x; v[k][1] += f0.y; v[k][2] += f1.x; v[k][3] += f1.y;
        }
      }
    }
  }
  if (trace) g_tp_trace[2] = global_timer_ns();
  // ---- residual, bf16 residual stream, RMSNorm: everything local from here on
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NP; ++k) {
    const int i = threadIdx.x + k * LL_THREADS;
    if (i < pairs) {
      if (res != nullptr) {
        const float2 f0 = unpack_bf16x2(res_v[k].x), f1 = unpack_bf16x2(res_v[k].y);
        v[k][0] += f0.x; v[k][1] += f0.y; v[k][2] += f1.x; v[k][3] += f1.y;
      }
      uint2 hv;
      hv.x = pack_bf16x2(v[k][0], v[k][1]);
      hv.y = pack_bf16x2(v[k][2], v[k][3]);
      const float2 f0 = unpack_bf16x2(hv.x), f1 = unpack_bf16x2(hv.y);
      v[k][0] = f0.x; v[k][1] = f0.y; v[k][2] = f1.x; v[k][3] = f1.y;
      ss += f0.x * f0.x + f0.y * f0.y + f1.x * f1.x + f1.y * f1.y;
      if (h_off >= 0) reinterpret_cast<uint2*>(own + h_off + static_cast<long long>(row) * d * 2)[i] = hv;
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) warp_ss[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int k = 0; k < LL_THREADS / 32; ++k) tot += warp_ss[k];
  const float rstd = rsqrtf(tot / static_cast<float>(d) + eps);
#pragma unroll
  for (int k = 0; k < NP; ++k) {
    const int i = threadIdx.x + k * LL_THREADS;
    if (i < pairs) {
      const float2 b0 = unpack_bf16x2(w_v[k].x), b1 = unpack_bf16x2(w_v[k].y);
      uint2 o;
      o.x = pack_bf16x2(v[k][0] * rstd * b0.x, v[k][1] * rstd * b0.y);
      o.y = pack_bf16x2(v[k][2] * rstd * b1.x, v[k][3] * rstd * b1.y);
      reinterpret_cast<uint2*>(own + y_off + static_cast<long long>(row) * d * 2)[i] = o;
    }
  }
  // every block read state[2] before it got here; the last one through advances the call number
  if (threadIdx.x == 0 && atomicAdd(&state[1], 1u) == gridDim.x - 1u) {
    state[1] = 0u;
    state[2] = epoch;
  }
}

// Block [B, n_loc] bf16 at column rank*n_loc of the row-major [B, ld] buffer at `buf_off`: copy it from this
// rank's region into every peer's, then wait until all peers' blocks are here.
template <bool MC>
__global__ void __launch_bounds__(256)
tp_allgather_cols_kernel(TpComm c, long long buf_off, int B, int n_loc, int ld, long long flag_off,
                         unsigned* __restrict__ state, unsigned long long timeout_ns, int* status) {
  griddep_launch();
  griddep_wait();
  if (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) return;   // an earlier wait ran out: stand down
  const unsigned epoch = state[0] + 1u;
  const int vec_per_row = n_loc >> 3;
  const long long total = static_cast<long long>(B) * vec_per_row;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(idx / vec_per_row), j = static_cast<int>(idx % vec_per_row);
    const long long off = buf_off + (static_cast<long long>(r) * ld + static_cast<long long>(c.rank) * n_loc + j * 8) * 2;
    uint32_t a[4];
    const uint4 q = *reinterpret_cast<const uint4*>(static_cast<const char*>(c.peer[c.rank]) + off);
    a[0] = q.x; a[1] = q.y; a[2] = q.z; a[3] = q.w;
    if constexpr (MC) {
      mc_st_16(static_cast<char*>(c.mc) + off, a);
    } else {
      for (int p = 0; p < c.world; ++p)
        if (p != c.rank) peer_st_16(static_cast<char*>(c.peer[p]) + off, a);
    }
  }
  __threadfence_system();
  __syncthreads();
  __shared__ unsigned last;
  if (threadIdx.x == 0) last = (atomicAdd(&state[1], 1u) == gridDim.x - 1u) ? 1u : 0u;
  __syncthreads();
  if (last) {
    exchange_flags(c, flag_off + RPEG_MAX_PEERS * 4, epoch, timeout_ns, status, 710);
    __syncthreads();
    if (threadIdx.x == 0) {
      state[1] = 0u;
      state[0] = epoch;
    }
  }
}

static int fill_comm(TpComm& c, void* const* peers, void* mc, int rank, int world) {
  if (world < 1 || world > RPEG_MAX_PEERS || rank < 0 || rank >= world) return -2;
  for (int i = 0; i < RPEG_MAX_PEERS; ++i) c.peer[i] = i < world ? peers[i] : nullptr;
  c.mc = mc;
  c.rank = rank;
  c.world = world;
  return 0;
}

}  // namespace rpeg

using namespace rpeg;

// peers: host array of `world` device addresses (the regions' bases, rank order); mc: multicast address or null.
// Offsets are bytes inside the region and multiples of 16; flag_off needs 2 * RPEG_MAX_PEERS uint32.
extern "C" int rpeg_tp_allreduce_rmsnorm(void* const* peers, void* mc, int rank, int world, long long part_off,
                                         const void* res, const void* w, long long y_off, long long h_off, int B, int d,
                                         float eps, long long flag_off, unsigned* state, unsigned long long timeout_ns,
                                         int* status, void* stream_v) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  TpComm c;
  if (fill_comm(c, peers, mc, rank, world)) return -2;
  if ((d & 7) || ((part_off | y_off | flag_off) & 15) || (h_off >= 0 && (h_off & 15))) return -3;
  if (B <= 0) return 0;
  const int rows_per = (B + world - 1) / world;
  const int nv = ((d >> 3) + 255) / 256;
  const __nv_bfloat16 *rp = static_cast<const __nv_bfloat16*>(res), *wp = static_cast<const __nv_bfloat16*>(w);
#define RPEG_TP_AR(NV_)                                                                                                   \
  do {                                                                                                                    \
    if (mc != nullptr)                                                                                                    \
      launch_pdl(tp_allreduce_rmsnorm_kernel<NV_, true>, dim3(rows_per), dim3(256), 0, stream, c, part_off, rp, wp, y_off, \
                 h_off, B, d, eps, flag_off, state, timeout_ns, status);                                                   \
    else                                                                                                                  \
      launch_pdl(tp_allreduce_rmsnorm_kernel<NV_, false>, dim3(rows_per), dim3(256), 0, stream, c, part_off, rp, wp, y_off, \
                 h_off, B, d, eps, flag_off, state, timeout_ns, status);                                                   \
  } while (0)
  if (nv == 1) RPEG_TP_AR(1);
  else if (nv == 2) RPEG_TP_AR(2);
  else if (nv <= 4) RPEG_TP_AR(4);
  else return -4;
#undef RPEG_TP_AR
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

extern "C" int rpeg_tp_allgather_cols(void* const* peers, void* mc, int rank, int world, long long buf_off, int B, int n_loc,
                                      int ld, long long flag_off, unsigned* state, unsigned long long timeout_ns, int* status,
                                      void* stream_v) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  TpComm c;
  if (fill_comm(c, peers, mc, rank, world)) return -2;
  if ((n_loc & 7) || (ld & 7) || ((buf_off | flag_off) & 15)) return -3;
  if (B <= 0 || n_loc <= 0) return 0;
  const long long total = static_cast<long long>(B) * (n_loc >> 3);
  const int grid = static_cast<int>(total / 256 < 1 ? 1 : (total / 256 > 148 ? 148 : total / 256));
  if (mc != nullptr)
    launch_pdl(tp_allgather_cols_kernel<true>, dim3(grid), dim3(256), 0, stream, c, buf_off, B, n_loc, ld, flag_off, state,
               timeout_ns, status);
  else
    launch_pdl(tp_allgather_cols_kernel<false>, dim3(grid), dim3(256), 0, stream, c, buf_off, B, n_loc, ld, flag_off, state,
               timeout_ns, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

// The one-shot variant: B <= ll_rows rows; the region holds 2 * world * ll_rows * d * 4 bytes of slots from ll_off
// (zero before the first call); state[2] counts the calls. d must be a multiple of 4.
extern "C" int rpeg_tp_allreduce_rmsnorm_ll(void* const* peers, void* mc, int rank, int world, long long part_off,
                                            const float* parts, int splits, long long split_stride, const void* res, const void* w, long long y_off, long long h_off, int B, int d,
                                            float eps, long long ll_off, int ll_rows, unsigned* state,
                                            unsigned long long timeout_ns, int* status, void* stream_v) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  TpComm c;
  if (fill_comm(c, peers, mc, rank, world)) return -2;
  if ((d & 7) || ((part_off | y_off | ll_off) & 15) || (h_off >= 0 && (h_off & 15))) return -3;
  if (B <= 0) return 0;
  if (B > ll_rows) return -5;
  if (parts != nullptr && (splits < 1 || (reinterpret_cast<uintptr_t>(parts) & 15) || (split_stride & 3))) return -6;
  const int np = ((d >> 2) + LL_THREADS - 1) / LL_THREADS;
  const __nv_bfloat16 *rp = static_cast<const __nv_bfloat16*>(res), *wp = static_cast<const __nv_bfloat16*>(w);
#define RPEG_TP_LL(NP_)                                                                                                     \
  do {                                                                                                                      \
    if (mc != nullptr)                                                                                                      \
      launch_pdl(tp_allreduce_rmsnorm_ll_kernel<NP_, true>, dim3(B), dim3(LL_THREADS), 0, stream, c, part_off, parts, splits, split_stride, rp, wp, y_off, h_off, \
                 B, d, eps, ll_off, ll_rows, state, timeout_ns, status);                                                     \
    else                                                                                                                    \
      launch_pdl(tp_allreduce_rmsnorm_ll_kernel<NP_, false>, dim3(B), dim3(LL_THREADS), 0, stream, c, part_off, parts, splits, split_stride, rp, wp, y_off, h_off, \
                 B, d, eps, ll_off, ll_rows, state, timeout_ns, status);                                                     \
  } while (0)
  if (np <= 1) RPEG_TP_LL(1);
  else if (np <= 2) RPEG_TP_LL(2);
  else if (np <= 4) RPEG_TP_LL(4);
  else return -4;
#undef RPEG_TP_LL
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

// Time stamps of the last traced launch of the one-shot all-reduce (block 0): ns from its start to the end of the push
// and to the moment all senders' units of the row were complete. enable != 0 switches the stamps on.
extern "C" int rpeg_tp_trace(int enable, unsigned long long* out2) {
  if (out2 != nullptr) {
    unsigned long long h[4];
    if (cudaMemcpyFromSymbol(h, g_tp_trace, sizeof(h)) != cudaSuccess) return -22;
    out2[0] = h[1] - h[0];
    out2[1] = h[2] - h[0];
  }
  const int on = enable ? 1 : 0;
  return cudaMemcpyToSymbol(g_tp_trace_on, &on, sizeof(on)) == cudaSuccess ? 0 : -22;
}
