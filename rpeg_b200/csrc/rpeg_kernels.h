// C ABI of librpeg_kernels.so (sm_100a). Every function enqueues work on `stream` (a cudaStream_t
// passed as void*) and returns 0 on success or a negative argument/launch error code; nothing here
// synchronises the device. Kernels that wait on barriers take an `int status[4]` device word
// {code, where, block, extra} that stays 0 unless a bounded wait ran out.
#pragma once
#include <stdint.h>

#define RPEG_MAX_PEERS 8
#define RPEG_KV_PAGE 64

#ifdef __cplusplus
extern "C" {
#endif

// ---- gemm.cu
int rpeg_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                   int transA, int transB, int out_fp32, int accumulate, int bn_hint, float* workspace,
                   long long workspace_elems, int* status, void* stream);
// Same GEMM, but no operand is read before gate_flags[0..gate_words) all reached min_version (bounded wait).
int rpeg_gemm_bf16_gated(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                         int transA, int transB, int out_fp32, int accumulate, int bn_hint, float* workspace,
                         long long workspace_elems, const unsigned* gate_flags, int gate_words, unsigned min_version,
                         unsigned long long timeout_ns, int* status, void* stream);

// ---- norm_rope.cu
int rpeg_rmsnorm_fwd(const void* x, const void* res, const void* w, void* h_out, void* y, float* rstd, int T,
                     int d, float eps, void* stream);
int rpeg_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres_in,
                     void* dx, float* dw, int T, int d, void* stream);
int rpeg_headnorm_fwd(void* buf, int ld, int col0, int nheads, int hd, const void* w, float* rstd, int T, float eps,
                      void* stream);
int rpeg_headnorm_bwd(void* dbuf, int ldd, const void* x, int ldx, int col0, int nheads, int hd, const void* w,
                      const float* rstd, float* dw, int T, void* stream);
// consumers of split-K partials: parts is fp32 [splits][rows][width], `stride` elements between splits
int rpeg_gemm_bf16_partials(const void* A, const void* B, int M, int N, int K, int lda, int ldb, float* workspace,
                            long long workspace_elems, int* k_splits_out, int* status, void* stream);
int rpeg_rmsnorm_fwd_partials(const float* parts, int splits, long long stride, const void* res, const void* w, void* h_out,
                              void* y, int T, int d, float eps, void* stream);
int rpeg_swiglu_fwd_partials(const float* parts, int splits, long long stride, void* out, long long T, int f, void* stream);
int rpeg_rope_kv_append_partials(const float* parts, int splits, long long stride, void* qkv, int ld, int q_col0, int k_col0,
                                 int v_col0, const int* seq_id, const int* pos, const float* cos_t, const float* sin_t,
                                 const int* page_table, int max_pages, void* kcache, void* vcache, int T, int H, int Hkv,
                                 int hd, void* stream);
int rpeg_rope(void* buf, const int* pos, const float* cos_t, const float* sin_t, int T, int ld, int col0,
              int nheads, int hd, int backward, void* stream);
int rpeg_swiglu_fwd(const void* gu, void* out, long long T, int f, void* stream);
int rpeg_swiglu_bwd(const void* gu, const void* dout, void* dgu, long long T, int f, void* stream);
int rpeg_add_bf16(const void* a, const void* b, void* out, long long n, void* stream);
int rpeg_embed_fwd(const int* ids, const void* table, void* out, int T, int d, void* stream);
int rpeg_embed_bwd(const int* ids, const void* dout, float* dtable, int T, int d, void* stream);

// ---- loss.cu
int rpeg_token_logprob_fwd(const void* logits, const int* targets, float* logp, float* lse, int T, int V,
                           int ld, float temperature, void* stream);
int rpeg_token_logprob_bwd(void* logits, const int* targets, const float* lse, const float* coef, int T,
                           int V, int ld, float temperature, void* stream);
int rpeg_token_entropy(const void* logits, const float* lse, float* ent, int T, int V, int ld, float temperature,
                       void* stream);
int rpeg_token_logprob_entropy_bwd(void* logits, const int* targets, const float* lse, const float* coef,
                                   const float* ent, const float* ecoef, int T, int V, int ld, float temperature,
                                   void* stream);
int rpeg_policy_loss(const float* lp, const float* old_lp, const float* ref_lp, const float* adv,
                     const float* mask, float* coef, float* acc, long long n, float clip_eps, float kl_coef,
                     float inv_denom, void* stream);
int rpeg_masked_rowsum(const float* x, const float* mask, float* out, int B, int T, void* stream);
int rpeg_dpo_loss(const float* pi_seq, const float* ref_seq, float* seq_coef, float* acc, int P, float beta,
                  void* stream);
int rpeg_expand_seq_coef(const float* seq_coef, const float* mask, float* coef, int B, int T, void* stream);
int rpeg_value_loss(const float* v, const float* ret, const float* mask, float* dv, float* acc, long long n,
                    float inv_denom, void* stream);
int rpeg_gae(const float* old_lp, const float* ref_lp, const float* values, const float* mask,
             const float* scores, float* adv, float* ret, int B, int T, float beta, float gamma, float lambda,
             int whiten, void* stream);
int rpeg_group_advantage(const float* rewards, float* out, int G, int K, void* stream);
int rpeg_sample(const void* logits, int B, int V, int ld, float temperature, int greedy,
                unsigned long long seed, const unsigned long long* seed_offset, const int* forced, int* token_out,
                float* logp_out, void* stream);
int rpeg_sample_filtered(const void* logits, int B, int V, int ld, float temperature, int top_k, float top_p,
                         unsigned long long seed, const unsigned long long* seed_offset, const int* forced, int* token_out,
                         float* logp_out, void* stream);
int rpeg_head_gemv(const void* h, const void* w, const float* bias, float* out, int T, int d, void* stream);
int rpeg_head_gemv_bwd(const void* h, const void* w, const float* dout, void* dh, float* dw, float* db, int T,
                       int d, void* stream);

// ---- optim.cu
int rpeg_adamw(float* p32, float* m, float* v, const float* grad, void* w16, long long n, float lr, float beta1,
               float beta2, float eps, float wd, int step, float grad_scale, const float* sumsq, int n_partials,
               float max_norm, void* stream);
int rpeg_sumsq(const float* x, long long n, float* out, void* stream);
int rpeg_flag_barrier(void* const* pads, int rank, int world, int slot, unsigned epoch, const float* payload_in,
                      float* payload_out, unsigned long long timeout_ns, int* status, void* stream);
int rpeg_dp_reduce_norm(void* const* grads, int world, long long shard_off, long long shard_n, float scale,
                        float* reduced, float* sumsq, void* stream);
int rpeg_dp_adam_push(float* p32, float* m, float* v, const float* reduced, void* const* params, int world,
                      long long shard_off, long long shard_n, float lr, float beta1, float beta2, float eps,
                      float wd, int step, const float* sumsq, int n_partials, float max_norm, void* stream);
int rpeg_copy16(const void* src, void* dst, long long nbytes, void* stream);
int rpeg_scatter_rows_by_index(const void* src, long long n, long long row_bytes, const long long* global_idx,
                               long long rows_per_rank, void* const* dst, int world, void* stream);
// Version words of pushed data: release-store `version` into word `word` of every destination flag array after
// the copies queued before it; poll flags[0..n) >= min_version with a bound (result[0] = 1 reached, 0 not yet).
// Programmatic dependent launches on/off for subsequent launches (graphs keep the setting of their capture).
void rpeg_set_pdl(int on);
int rpeg_publish_version(void* const* flag_arrays, int n_dst, int word, unsigned version, void* stream);
int rpeg_wait_flags(const unsigned* flags, int n, unsigned min_version, unsigned long long timeout_ns, int* result,
                    void* stream);
int rpeg_copy2d(const void* src, long long src_pitch, void* dst, long long dst_pitch, long long rows, long long row_bytes,
                void* stream);

// ---- gemm_rs.cu: row-parallel linear = GEMM + reduce-scatter (or all-reduce) over peer memory in one launch
int rpeg_gemm_rs(const void* A, const void* B, int M, int N, int K, int lda, int ldb, void* const* stage,
                 void* const* counters, void* const* outs, int ldo, int rank, int world, unsigned epoch, int all_gather,
                 int* status, void* stream);

// ---- ag_gemm.cu: column-parallel linear = all-gather of the activation rows + GEMM in one launch
int rpeg_ag_gemm(void* const* xs, const void* W, void* Y, void* const* readys, int M, int N, int K, int ldx, int ldw, int ldy,
                 int rank, int world, unsigned epoch, int* status, void* stream);

// ---- decode_attn.cu
int rpeg_kv_append(const void* qkv, int ld, int k_col0, int v_col0, const int* seq_id, const int* pos,
                   const int* page_table, int max_pages, void* kcache, void* vcache, int T, int Hkv, int hd,
                   void* stream);
int rpeg_rope_kv_append(void* qkv, int ld, int q_col0, int k_col0, int v_col0, const int* seq_id, const int* pos,
                        const float* cos_t, const float* sin_t, const int* page_table, int max_pages, void* kcache,
                        void* vcache, int T, int H, int Hkv, int hd, void* stream);
long long rpeg_decode_attn_scratch_bytes(int B, int H, int nsplit);
int rpeg_paged_decode_attn(const void* q, int ldq, int q_col0, const void* kcache, const void* vcache,
                           const int* page_table, int max_pages, const int* seq_lens, void* out, float* scratch,
                           int B, int H, int Hkv, int hd, int nsplit, float scale, void* stream);
// Same, for batches whose rows share their first keys in groups (page-table aliasing): group_rows [B, 8], group_shared [B],
// row_key0 [B]; scratch sized for nsplit + 1 partials.
int rpeg_paged_decode_attn_grouped(const void* q, int ldq, int q_col0, const void* kcache, const void* vcache,
                                   const int* page_table, int max_pages, const int* seq_lens, void* out, float* scratch,
                                   int B, int H, int Hkv, int hd, int nsplit, float scale, const int* group_rows,
                                   const int* group_shared, const int* row_key0, void* stream);

// ---- symm.cu
int rpeg_symm_alloc(unsigned long long bytes, void** out);
int rpeg_symm_free(void* p);
int rpeg_ipc_export(void* p, void* handle64);
int rpeg_ipc_open(const void* handle64, void** out);
int rpeg_ipc_close(void* p);
int rpeg_memset_async(void* p, int value, unsigned long long bytes, void* stream);

// ---- generate.cu
int rpeg_decode_prepare(const int* active, const int* gen_count, const int* forced_len, int* forced, int n_slots,
                        int eos, void* stream);
int rpeg_decode_advance(const int* sampled, const float* sampled_lp, int* token, int* pos, int* seq_len,
                        int* active, int* gen_count, int* out_tok, float* out_lp, int n_slots, int max_new,
                        int eos, int* n_finished, unsigned long long* step_counter, void* stream);
int rpeg_gather_rows(const void* x, const int* rows, void* out, int n, int d, void* stream);
int rpeg_scatter_rows(void* x, const int* rows, const void* src, int n, int d, int overwrite, void* stream);
int rpeg_splitk_reduce(const float* part, void* out, int M, int N, int ldc, int splits, void* stream);

// ---- flash_attn.cu
int rpeg_flash_attn_fwd(const void* qkv, int ld, int q_col0, int k_col0, int v_col0, const int* cu_seqlens,
                        int B, int max_seqlen, int T, int H, int Hkv, int hd, float scale, void* out, float* lse,
                        int* status, void* stream);

int rpeg_flash_attn_bwd(const void* qkv, int ld, int q_col0, int k_col0, int v_col0, const void* out,
                        const void* dout, const float* lse, const int* cu_seqlens, int B, int max_seqlen, int T,
                        int H, int Hkv, int hd, float scale, float* dvec, float* dq_acc, void* dqkv, int ld_dqkv,
                        int* status, void* stream);

#ifdef __cplusplus
}
#endif
