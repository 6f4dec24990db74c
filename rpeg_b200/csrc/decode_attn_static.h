// Split-KV paged decode attention that never allocates: its scratch is a fixed array inside the library.
//
// This entry point has no counterpart in the reference; it exists for callers of this library that
// cannot allocate device memory at the point of the call and cannot hand in a scratch buffer either:
// a host thread that drives a pre-built serving loop from C with a fixed memory budget, or code that
// runs while the process's allocator is locked down. The regular entry (rpeg_paged_decode_attn)
// takes its split-KV scratch from the caller, who usually gets it from an allocator.
//
// Limits and rules:
//   * B * H * nsplit must not exceed RPEG_DECODE_STATIC_MAX_PARTIALS (16384); each partial is 130 floats,
//     so the array is 16384 * 130 * 4 bytes = 8.1 MiB per device. Larger problems are refused with
//     RPEG_STATIC_ERR_TOO_LARGE; rpeg_static_entry_strerror() gives the text.
//   * The first call on a device (with that device current) looks the array's address up once with
//     cudaGetSymbolAddress and keeps it. Make that first call during start-up, before any stream
//     capture is begun on that device.
//   * Nothing in the scratch has to start at zero: every slot the combine pass reads was written by the
//     split pass of the same call.
//   * There is ONE array per device. Two calls whose kernels may overlap in time (different streams,
//     or different host threads) race on it; keep all calls on a device in one stream, or order them.
//   * No cudaMalloc / cudaFree and no allocating library routine is called, on the first call or later.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define RPEG_DECODE_STATIC_MAX_PARTIALS 16384
#define RPEG_STATIC_ERR_BAD_SHAPE (-2)
#define RPEG_STATIC_ERR_BAD_SPLIT (-3)
#define RPEG_STATIC_ERR_TOO_LARGE (-5)
#define RPEG_STATIC_ERR_SETUP (-6)
#define RPEG_STATIC_ERR_LAUNCH (-21)

// Same arguments and result as rpeg_paged_decode_attn without the scratch pointer (1 <= nsplit <= 64).
int rpeg_paged_decode_attn_static(const void* q, int ldq, int q_col0, const void* kcache, const void* vcache,
                                  const int* page_table, int max_pages, const int* seq_lens, void* out, int B, int H,
                                  int Hkv, int hd, int nsplit, float scale, void* stream);

// Human-readable text for the codes above (a static string; never NULL).
const char* rpeg_static_entry_strerror(int code);

#ifdef __cplusplus
}
#endif
