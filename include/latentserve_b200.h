/* latentserve_b200 — C ABI of the sm_100a paged decode-attention kernels.
 *
 * One shared library (libls_b200.so), plain pointers and sizes, no PyTorch
 * types. Every pointer is a DEVICE pointer unless stated; every stride is in
 * ELEMENTS of the tensor it belongs to; `stream` is a cudaStream_t passed as
 * void* (0 = the default stream). Every entry point only validates and
 * launches: no allocation, no host synchronisation, no device-to-host copy, so
 * all of them can be recorded into a CUDA graph. The caller owns every buffer.
 *
 * Return value: 0 on success; < 0 an argument error (LS_ERR_*), nothing was
 * launched; > 0 the cudaError_t of a failed launch.
 *
 * Shapes use B = sequences in the batch, H = KV heads, R = query rows per KV
 * head (GQA ratio, <= 8), D = 128 (head_dim), P = 16 (tokens per page),
 * NB = blocks in the pool, MP = block-table width. Each declaration cites the
 * reference interface (path inside the LatentServe tree : lines) it replaces.
 */
#ifndef LATENTSERVE_B200_H
#define LATENTSERVE_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LS_OK 0
#define LS_ERR_NULL_POINTER (-1)
#define LS_ERR_BAD_SHAPE (-2)
#define LS_ERR_BAD_STRIDE (-3)
#define LS_ERR_MISALIGNED (-4)
#define LS_ERR_TOO_LARGE (-5)
#define LS_ERR_UNSUPPORTED (-6)
#define LS_ERR_SCRATCH_TOO_SMALL (-7)
#define LS_ERR_NOALLOC_LIMIT (-8) /* ls_paged_decode_fp16_noalloc: shape past its fixed scratch */
#define LS_NOALLOC_SCRATCH_BYTES 4264704

/* `flags` of the decode entry points. The low byte of ls_paged_decode_fp16's
 * flags picks the kernel variant. */
#define LS_IMPL_MMA 0  /* tensor-core kernel (the product path) */
#define LS_IMPL_SIMT 1 /* CUDA-core kernel, fp16 pools only (kept for profiling) */
/* Launch with programmatic stream serialization: the kernel may be scheduled
 * while the previous kernel of the stream is still draining, and it reads
 * seq_lens and block_tables (nothing else) before it synchronises on that
 * kernel. Only set it when the kernel launched just before on the stream does
 * not write seq_lens or block_tables (in LatentServe it is the KV append). */
#define LS_LAUNCH_PROGRAMMATIC 0x100
/* How the decode entry points bring pages into shared memory. By default the
 * INT8 kernel (pools in the standard layout) uses TMA tile copies issued
 * by one lane per warp -- it is instruction-issue bound and gains 14 % -- and the
 * fp16 kernels use per-lane cp.async, which measured 3 % faster on those
 * memory-bound kernels. LS_LOAD_CP_ASYNC / LS_LOAD_TMA force one form (TMA is not
 * available for the CUDA-core variant or for layouts a tensor map cannot describe:
 * the cp.async form runs then). Results are identical. */
#define LS_LOAD_CP_ASYNC 0x200
#define LS_LOAD_TMA 0x400
/* INT8 entry points, TMA loader: a page's K tile and V tile normally arrive by ONE tile
 * copy, through a tensor map that spans both pools (possible whenever the two allocations
 * lie less than 2^40 bytes apart). With this flag they are fetched by one copy each, which
 * is also what happens by itself when the pools are further apart. Results are identical. */
#define LS_LOAD_TMA_SPLIT_KV 0x1000
/* With LS_LAUNCH_PROGRAMMATIC on the dense entry points (fp16, INT8): also request
 * the first pages before synchronising on the previous kernel of the stream, except
 * a sequence's LAST page (the one holding token seq_len - 1), which is requested
 * after it; with INT8 pools the page before the last is held back as well, because
 * an INT8 cache quantises a K page in the step after the one that filled it. Only set
 * it when nothing that runs between the previous step's attention and this launch
 * writes the pools (pages, scales, zero points) outside those pages -- in LatentServe
 * that is the KV append (the newest token) and, for INT8, the page finalisation. */
#define LS_EARLY_PAGES 0x800

/* Partial-state scratch shared by the three decode entry points.
 *
 * The batch's pages are cut into `num_chunks` equal chunks; each (chunk,
 * sequence) piece writes one partial softmax state. With
 * slots = ls_decode_slots(B, num_chunks) the caller provides
 *   part_acc  float [slots, H, 8, 128]
 *   part_m    float [slots, H, 8]        running maxima, log2 domain
 *   part_l    float [slots, H, 8]
 *   seg_range int32 [2*B + 2 + B*H]      [0, 2B): first slot and slot count of
 *                                        each sequence, written by the kernel;
 *                                        [2B]: set to 1 if a block id or a
 *                                        residual row outside its pool was met
 *                                        (that page is skipped, never read);
 *                                        [2B+2, ...): one arrival counter per
 *                                        (sequence, head), left at zero by
 *                                        every launch. ZERO THE BUFFER ONCE
 *                                        before first use.
 * None of it needs filling between calls. `num_chunks` x H is the grid: the
 * fp16 kernels are sized for 2 resident CTAs per SM and the INT8 kernels for
 * 4, so num_chunks = 2*SMs / H (3*SMs / H for INT8) is the natural choice; `min_chunk` (>= 1) is the fewest pages a chunk may hold.
 * If `out` is non-NULL the same launch also merges the partials — the CTA that
 * delivers a sequence's last partial does it, nobody waits — and `out`
 * receives fp16 [B, H, R, 128] with the given strides; sequences of length 0
 * get zeros. If `out` is NULL only the partials are produced (ls_combine
 * merges them). Launches that share one scratch must not overlap on the GPU.
 */
int ls_decode_slots(int batch, int num_chunks);

/* Dense fp16 paged GQA decode attention, split-KV partials (+ merge).
 * Replaces kernels/cuda/paged_decode_fp16.cu:55-200 (kernel `paged_decode_fp16`)
 * as launched by kernels/cuda/paged_decode_cuda.py:202-252.
 *   q [B,H,R,128] fp16 (sq_*), k_pool/v_pool [NB,16,H,128] fp16 (sk_b, sk_p, sk_h; same for both),
 *   block_tables int32 rows of stride max_pages, seq_lens int32 [B].
 * Rows need 16-byte alignment. B <= 1024. */
int ls_paged_decode_fp16(const void* q, const void* k_pool, const void* v_pool,
                         const int32_t* block_tables, const int32_t* seq_lens, float* part_acc,
                         float* part_m, float* part_l, int32_t* seg_range, void* out, int batch,
                         int kv_heads, int n_rep, int head_dim, int page, int max_pages,
                         int num_blocks, int num_chunks, int min_chunk, int flags, int64_t sq_b,
                         int64_t sq_h, int64_t sq_m, int64_t sk_b, int64_t sk_p, int64_t sk_h,
                         int64_t so_b, int64_t so_h, int64_t so_m, float softmax_scale,
                         void* stream);

/* The same launch with the step's KV append riding on it: the new token's K and V rows
 * (the rows a decode step would first scatter into the pools) are handed to the attention
 * kernel, which takes the newest row of each sequence's last page from them, stores them to
 * the pools for the steps to come, and attends as if they had been appended first. One
 * launch per layer instead of two.
 * Replaces PagedKVCache.write (cache/paged_cache.py:398-417, two index_copy_) followed by
 * `paged_decode_fp16` (kernels/cuda/paged_decode_fp16.cu:55-200), as GQAAttention.forward
 * runs them back to back (model/attention/gqa.py:267, 283-344).
 *   k_new, v_new fp16 rows [B,H,128] (sn_b, sn_h / svn_b, svn_h), 16-byte aligned; the row of
 *   sequence b goes to position seq_lens[b] - 1, i.e. block_tables[b][(L-1)/16], row (L-1)%16.
 *   seq_lens already count the new token. Page bounds are not maintained by this entry
 *   point (use ls_kv_append_fp16 when the sparse indexer is on). Per-lane copies only
 *   (LS_LOAD_TMA is ignored). */
int ls_paged_decode_append_fp16(const void* q, const void* k_new, const void* v_new, void* k_pool,
                                void* v_pool, const int32_t* block_tables, const int32_t* seq_lens,
                                float* part_acc, float* part_m, float* part_l, int32_t* seg_range, void* out,
                                int batch, int kv_heads, int n_rep, int head_dim, int page, int max_pages,
                                int num_blocks, int num_chunks, int min_chunk, int flags, int64_t sq_b,
                                int64_t sq_h, int64_t sq_m, int64_t sn_b, int64_t sn_h, int64_t svn_b,
                                int64_t svn_h, int64_t sk_b, int64_t sk_p, int64_t sk_h, int64_t so_b,
                                int64_t so_h, int64_t so_m, float softmax_scale, void* stream);

/* Dense fp16 decode for callers that cannot allocate device memory. No
 * counterpart in the reference (its scratch comes from torch's allocator,
 * kernels/gqa/paged_decode.py:501-517, and every caller there has one).
 *
 * Same computation and arguments as ls_paged_decode_fp16 with the tensor-core
 * kernel, minus the four scratch pointers: the partial states live in a fixed
 * array inside the library image (LS_NOALLOC_SCRATCH_BYTES, about 4.1 MiB of
 * device memory on every GPU that loads the library, held until exit). Meant
 * for hosts that reach this ABI through an FFI and own no device allocator,
 * and for processes that gave all device memory away at start-up, where a
 * cudaMalloc on the decode path may fail and stalls the device while it runs.
 *   Limits: batch <= 64 and (batch + num_chunks) * kv_heads <= 1024, else
 *   LS_ERR_NOALLOC_LIMIT and nothing is launched. `out` is required.
 *   The first call on a device resolves the array's device address
 *   (cudaGetSymbolAddress, with that device current): make it before any
 *   stream capture starts. The address is remembered per device ordinal for the
 *   life of the process and does not survive a cudaDeviceReset; `stream` must
 *   belong to the device that is current at the call. Calls share the array: its
 *   bookkeeping part is cleared on `stream` at the start of every call, and calls
 *   whose kernels overlap on one GPU race — keep them ordered. Allocates nothing.
 *   Block ids are checked against num_blocks on the device and a page with an id
 *   outside the pool is skipped, never read; the word that records such a skip
 *   lives in the built-in array and this entry point offers no way to read it, so
 *   a caller with an untrusted block table validates it on the host (the ordinary
 *   entry point reports it in seg_range[2B]). */
int ls_paged_decode_fp16_noalloc(const void* q, const void* k_pool, const void* v_pool,
                                 const int32_t* block_tables, const int32_t* seq_lens, void* out,
                                 int batch, int kv_heads, int n_rep, int head_dim, int page,
                                 int max_pages, int num_blocks, int num_chunks, int min_chunk,
                                 int64_t sq_b, int64_t sq_h, int64_t sq_m, int64_t sk_b, int64_t sk_p,
                                 int64_t sk_h, int64_t so_b, int64_t so_h, int64_t so_m,
                                 float softmax_scale, void* stream);

/* INT8 paged GQA decode attention.
 * Replaces kernels/cuda/paged_decode_int8.cu:87-280 (kernel `paged_decode_int8`,
 * variants ASYM / HAS_RES) as launched by kernels/cuda/paged_decode_cuda.py:202-252.
 *   k_pool/v_pool [NB,16,H,128] int8; k_scale (and k_zero) float [NB,H,128] (ks_b, ks_h);
 *   v_scale (and v_zero) float [NB,16,H] (vs_b, vs_p, vs_h); k_zero/v_zero both NULL = symmetric;
 *   k_res fp16 [rows,16,H,128] (sr_r, sr_p, sr_h) with res_rows int32 [B]: each sequence's LAST
 *   page of K is read from k_res[res_rows[b]] instead of the pool (both NULL = no residual). */
int ls_paged_decode_int8(const void* q, const void* k_pool, const void* v_pool,
                         const int32_t* block_tables, const int32_t* seq_lens, const float* k_scale,
                         const float* v_scale, const float* k_zero, const float* v_zero,
                         const void* k_res, const int32_t* res_rows, float* part_acc, float* part_m,
                         float* part_l, int32_t* seg_range, void* out, int batch, int kv_heads,
                         int n_rep, int head_dim, int page, int max_pages, int num_blocks,
                         int num_res_rows, int num_chunks, int min_chunk, int flags, int64_t sq_b,
                         int64_t sq_h, int64_t sq_m, int64_t sk_b, int64_t sk_p, int64_t sk_h,
                         int64_t ks_b, int64_t ks_h, int64_t vs_b, int64_t vs_p, int64_t vs_h,
                         int64_t sr_r, int64_t sr_p, int64_t sr_h, int64_t so_b, int64_t so_h,
                         int64_t so_m, float softmax_scale, void* stream);

/* INT8 pools, attention over the pages in `sel` only: ls_paged_decode_int8 with the
 * page-list arguments of ls_paged_sparse_fp16 in front (symmetric pools only). The
 * reference has no such kernel (its sparse path is fp16 only,
 * docs/phase16_int8_sparse.md:21-26); here it is one more instance of the same
 * decode kernel. A selected page that is the sequence's last takes its K from the
 * fp16 residual, as in the dense INT8 kernel. */
int ls_paged_sparse_int8(const int32_t* sel, float ratio, int recent, int num_sel, int64_t sl_b,
                         int64_t sl_h, const void* q, const void* k_pool, const void* v_pool,
                         const int32_t* block_tables, const int32_t* seq_lens, const float* k_scale,
                         const float* v_scale, const float* k_zero, const float* v_zero,
                         const void* k_res, const int32_t* res_rows, float* part_acc, float* part_m,
                         float* part_l, int32_t* seg_range, void* out, int batch, int kv_heads,
                         int n_rep, int head_dim, int page, int max_pages, int num_blocks,
                         int num_res_rows, int num_chunks, int min_chunk, int flags, int64_t sq_b,
                         int64_t sq_h, int64_t sq_m, int64_t sk_b, int64_t sk_p, int64_t sk_h,
                         int64_t ks_b, int64_t ks_h, int64_t vs_b, int64_t vs_p, int64_t vs_h,
                         int64_t sr_r, int64_t sr_p, int64_t sr_h, int64_t so_b, int64_t so_h,
                         int64_t so_m, float softmax_scale, void* stream);

/* Attention over selected pages only.
 * Replaces kernels/cuda/paged_sparse_fp16.cu:205-364 (kernel `paged_sparse_fp16`)
 * as launched by kernels/cuda/paged_sparse.py:185-219.
 *   sel int32 [B,H,num_sel] (sl_b, sl_h): page indices, best first. With ratio > 0 each sequence
 *   attends the first n = min(max(recent+1, ceil(ratio*pages)), pages, num_sel) entries
 *   (pages = its own page count; ratio >= 1: all its pages); ratio <= 0: every entry.
 *   Entries < 0 or >= pages are skipped. */
int ls_paged_sparse_fp16(const void* q, const void* k_pool, const void* v_pool,
                         const int32_t* block_tables, const int32_t* seq_lens, const int32_t* sel,
                         float ratio, int recent, float* part_acc, float* part_m, float* part_l,
                         int32_t* seg_range, void* out, int batch, int kv_heads, int n_rep,
                         int head_dim, int page, int max_pages, int num_blocks, int num_sel,
                         int num_chunks, int min_chunk, int flags, int64_t sq_b, int64_t sq_h,
                         int64_t sq_m, int64_t sk_b, int64_t sk_p, int64_t sk_h, int64_t sl_b,
                         int64_t sl_h, int64_t so_b, int64_t so_h, int64_t so_m, float softmax_scale,
                         void* stream);

/* Merge of the split partials into out fp16 [B,H,R,128].
 * Replaces the Triton `_combine_kernel`, kernels/gqa/paged_decode.py:421-471
 * (torch form `combine_splits`, :689-706). Reads seg_range as a decode entry
 * point left it. */
int ls_combine(const float* part_acc, const float* part_m, const float* part_l,
               const int32_t* seg_range, void* out, int batch, int kv_heads, int n_rep,
               int64_t so_b, int64_t so_h, int64_t so_m, void* stream);

/* fp16 cache append for one new token per sequence: K and V rows scattered to
 * flat slot `slots[b]` of the pools and, if kmin/kmax are given, the page's
 * per-channel K bounds reset (slot % 16 == 0) or widened.
 * Replaces PagedKVCache.write, cache/paged_cache.py:398-417 (two index_copy_) and
 * `page_bounds_update`, kernels/cuda/paged_sparse_fp16.cu:54-72.
 *   k, v fp16 rows [B,H,128] (sk_b, sk_h / sv_b, sv_h); slots int64 [B];
 *   k_pool/v_pool viewed flat [num_slots,H,128] (sp_t, sp_h); kmin/kmax fp16 [NB,H,128] (sb_b, sb_h).
 *   k_pool == v_pool == NULL: bounds only. */
int ls_kv_append_fp16(const void* k, const void* v, const int64_t* slots, void* k_pool, void* v_pool,
                      void* kmin, void* kmax, int batch, int kv_heads, int head_dim, int page,
                      int64_t num_slots, int64_t sk_b, int64_t sk_h, int64_t sv_b, int64_t sv_h,
                      int64_t sp_t, int64_t sp_h, int64_t sb_b, int64_t sb_h, void* stream);

/* INT8 cache decode-step write: V quantised per (token, head) and scattered,
 * K copied into the fp16 residual. Bit-exact with the reference.
 * Replaces `int8_decode_write`, kernels/cuda/int8_write.cu:45-78
 * (host side kernels/cuda/int8_write.py:61-81).
 *   flat_v int8 [num_slots,H,128], flat_v_scale / flat_v_zero float [num_slots,H],
 *   k_res fp16 [num_res,H,128], all contiguous; res_idx int64 [B] rows of k_res.
 *   inv_qmax = (float)1 / (float)qmax and inv_levels likewise, formed by the caller. */
int ls_int8_decode_write(const void* k, const void* v, const int64_t* slots, const int64_t* res_idx,
                         void* flat_v, float* flat_v_scale, float* flat_v_zero, void* k_res,
                         int batch, int kv_heads, int head_dim, int64_t num_slots, int64_t num_res,
                         int64_t sk_b, int64_t sk_h, int64_t sv_b, int64_t sv_h, int asym, float eps,
                         float qmax, float inv_qmax, float levels, float inv_levels, float offset,
                         void* stream);

/* INT8 cache: quantise completed K pages out of the residual, one step per
 * (block, head, channel). Bit-exact with the reference's torch ops on a GPU.
 * Replaces Int8PagedKVCache._finalize_blocks, cache/int8_paged_cache.py:670-699.
 *   k_res fp16 [num_rows,16,H,128] (sr_*); res_rows / block_ids int64 [count];
 *   k_pool int8 [NB,16,H,128] (sk_*); k_scale / k_zero float [NB,H,128] (ss_b, ss_h). */
int ls_int8_finalize_blocks(const void* k_res, const int64_t* res_rows, const int64_t* block_ids,
                            void* k_pool, float* k_scale, float* k_zero, int count, int kv_heads,
                            int head_dim, int page, int64_t num_rows, int64_t num_blocks,
                            int64_t sr_r, int64_t sr_p, int64_t sr_h, int64_t sk_b, int64_t sk_p,
                            int64_t sk_h, int64_t ss_b, int64_t ss_h, int asym, float eps, float qmax,
                            float inv_qmax, float levels, float inv_levels, float offset,
                            void* stream);

/* The same for `layers` layers in one launch, when the layers' residuals, pools and
 * scales are slices of stacked tensors: layer l's tensors start sr_l / sk_l / ss_l
 * elements after layer l-1's. The same residual rows go to the same blocks in every
 * layer (a sequence's page completes in all layers at once). */
int ls_int8_finalize_layers(const void* k_res, const int64_t* res_rows, const int64_t* block_ids,
                            void* k_pool, float* k_scale, float* k_zero, int count, int layers,
                            int kv_heads, int head_dim, int page, int64_t num_rows, int64_t num_blocks,
                            int64_t sr_l, int64_t sr_r, int64_t sr_p, int64_t sr_h, int64_t sk_l,
                            int64_t sk_b, int64_t sk_p, int64_t sk_h, int64_t ss_l, int64_t ss_b,
                            int64_t ss_h, int asym, float eps, float qmax, float inv_qmax, float levels,
                            float inv_levels, float offset, void* stream);

/* The same with the LENGTH of the page list on the device, so that the launch can be
 * a fixed node of a captured decode step and the host's per-step work for the INT8
 * cache is one staged copy and no launch. Replaces the eager torch ops that
 * Int8PagedKVCache.advance runs through _finalize_pending, outside the graph, on the
 * step's critical path (cache/int8_paged_cache.py:443-446, 524-552).
 *   state int32 [2] (device): state[0] = entries of res_rows / block_ids to finalise
 *   (written by the host's staged copy before the step), state[1] = 0. The grid is
 *   fixed by max_count (capacity of the lists). The list is consumed once: the kernel
 *   sets state[0] back to 0 when it is done, so replaying the step without a new list
 *   finalises nothing. Launch it before the step's first residual write. */
int ls_int8_finalize_pending(const void* k_res, const int64_t* res_rows, const int64_t* block_ids,
                             int32_t* state, void* k_pool, float* k_scale, float* k_zero,
                             int max_count, int layers, int kv_heads, int head_dim, int page,
                             int64_t num_rows, int64_t num_blocks, int64_t sr_l, int64_t sr_r,
                             int64_t sr_p, int64_t sr_h, int64_t sk_l, int64_t sk_b, int64_t sk_p,
                             int64_t sk_h, int64_t ss_l, int64_t ss_b, int64_t ss_h, int asym, float eps,
                             float qmax, float inv_qmax, float levels, float inv_levels, float offset,
                             void* stream);

/* Page scores for sparse selection: Quest upper bound from per-page K min/max,
 * maximised over the R query rows; +inf for page 0 and the `recent` last
 * pages, -inf past the sequence's end. fp32 evaluation order as the reference.
 * Replaces `page_index`, kernels/cuda/paged_sparse_fp16.cu:78-130
 * (host side kernels/cuda/paged_sparse.py:104-123).
 *   kmin/kmax fp16 [NB,H,128] (sb_b, sb_h); scores float [B,H,max_pages] (ss_b, ss_h);
 *   table_stride = block-table row stride >= max_pages. */
int ls_page_index(const void* q, const void* kmin, const void* kmax, const int32_t* block_tables,
                  const int32_t* seq_lens, float* scores, int batch, int kv_heads, int n_rep,
                  int head_dim, int page, int max_pages, int table_stride, int num_blocks,
                  int recent, int64_t sq_b, int64_t sq_h, int64_t sq_m, int64_t sb_b, int64_t sb_h,
                  int64_t ss_b, int64_t ss_h, void* stream);

/* ls_page_index followed by ls_select_pages (below) behind one call, with the launch
 * flags the other entry points take. Same scores, same selection.
 * Replaces `page_scores` + `select` as `sparse_attention` runs them back to back,
 * kernels/cuda/paged_sparse.py:222-251.
 *   scores float [B,H,max_pages] (written); sel int32 [B,H,k] (written).
 *   flags: LS_LAUNCH_PROGRAMMATIC, and with it LS_EARLY_PAGES: block ids and page bounds are
 *   requested before the index kernel synchronises on the previous kernel of the stream. Only
 *   set that when nothing between the previous step and this launch writes block_tables,
 *   seq_lens or the bounds of any page but a sequence's last (the bounds it reads are never a
 *   last page's, given recent >= 1; with recent == 0 the flag is ignored). (Folding the
 *   selection into the index kernel's last-arriving CTA per row was built and measured: a
 *   128-thread CTA selects slower than the 512-thread kernel does, 51 against 46 us per
 *   layer call at 8 x 32 768, so the two stay separate launches.) */
int ls_page_index_select(const void* q, const void* kmin, const void* kmax, const int32_t* block_tables,
                         const int32_t* seq_lens, float* scores, int32_t* sel, int batch, int kv_heads,
                         int n_rep, int head_dim, int page, int max_pages, int table_stride,
                         int num_blocks, int recent, int k, float ratio, int flags, int64_t sq_b,
                         int64_t sq_h, int64_t sq_m, int64_t sb_b, int64_t sb_h, int64_t ss_b, int64_t ss_h,
                         int64_t sl_b, int64_t sl_h, void* stream);

/* Per-query-row bounds float [B,H,R,max_pages] (sh_b, sh_h, sh_r), 0 past the end.
 * Replaces `page_index_heads`, kernels/cuda/paged_sparse_fp16.cu:141-190. */
int ls_page_index_heads(const void* q, const void* kmin, const void* kmax,
                        const int32_t* block_tables, const int32_t* seq_lens, float* heads_out,
                        int batch, int kv_heads, int n_rep, int head_dim, int page, int max_pages,
                        int table_stride, int num_blocks, int64_t sq_b, int64_t sq_h, int64_t sq_m,
                        int64_t sb_b, int64_t sb_h, int64_t sh_b, int64_t sh_h, int64_t sh_r,
                        void* stream);

/* Top-k pages per (sequence, KV head): sel int32 [B,H,k] (sl_b, sl_h), score
 * descending, ties to the lower page index. num_pages <= 8192 (a 128K context).
 * Replaces torch.topk(..., sorted=True) in `select`, kernels/cuda/paged_sparse.py:164-168. */
int ls_topk_pages(const float* scores, int32_t* sel, int batch, int kv_heads, int num_pages, int k,
                  int64_t ss_b, int64_t ss_h, int64_t sl_b, int64_t sl_h, void* stream);

/* Selection for the fused index -> select -> attend path, without the sort: for each
 * (sequence, head) the n pages with the highest scores, n = the sequence's own budget
 * from its own length (the rule ls_paged_sparse_* applies: max(recent + 1,
 * ceil(ratio x pages)), capped at its pages and at k; ratio <= 0 or >= 1: min(pages, k)),
 * ties to the lower page -- the same set as the first n entries ls_topk_pages returns --
 * written in ascending page order and followed by -1 up to k. A radix search for the
 * n-th largest score and two block scans; about half the time of the sort. No
 * counterpart in the reference (it sorts with torch.topk, kernels/cuda/paged_sparse.py:164-168,249). */
int ls_select_pages(const float* scores, const int32_t* seq_lens, int32_t* sel, int batch, int kv_heads,
                    int num_pages, int k, float ratio, int recent, int64_t ss_b, int64_t ss_h,
                    int64_t sl_b, int64_t sl_h, void* stream);

/* ---- The per-layer kernels around attention (the callers' side of the path) ---- */

/* RMSNorm over fp16 rows, optionally fused with the residual add:
 *   s = fp16(x + residual); res_out = s; y = fp16(weight * fp16(s * rsqrt(mean(s^2) + eps))).
 * residual == res_out == NULL: plain RMSNorm of x. n % 8 == 0, rows 16-byte aligned.
 * Replaces the Triton `_rms_norm_kernel`, kernels/fused_elementwise.py:118-137
 * (torch forms `rms_norm_ref` / `fused_add_rms_norm_ref`, :75-86). */
int ls_rms_norm(const void* x, const void* residual, const void* weight, void* y, void* res_out,
                int rows, int n, float eps, int64_t sx, int64_t sr, int64_t sy, int64_t sro,
                void* stream);

/* out[r, i] = fp16(fp16(silu(gate_up[r, i])) * gate_up[r, inter + i]), fp16 rows.
 * Replaces the Triton `_silu_mul_kernel`, kernels/fused_elementwise.py:140-151
 * (torch form `silu_and_mul_ref`, :89-91). */
int ls_silu_mul(const void* gate_up, void* out, int rows, int inter, int64_t sgu, int64_t sout,
                void* stream);

/* RoPE of the query and key heads of a fused QKV projection row, fused with the
 * KV append of the fp16 cache: one launch writes q_out [B, q_heads, 128] (rotated),
 * the rotated K row and the V row at flat slot slots[b] of the pools, and the
 * page's K bounds when kmin/kmax are given.
 *   qkv fp16 [B, (q_heads + 2 kv_heads) * 128] (row stride s_qkv), heads in q, k, v order;
 *   cos, sin fp16 [max_pos, 128] (row stride s_cos), halves duplicated; positions int64 [B].
 * Rounding as the reference's rope (three fp16 roundings per output).
 * Replaces the Triton `_rope_kernel`, kernels/fused_elementwise.py:154-182 (torch form
 * `rope_qk_ref`, :99-107) followed by PagedKVCache.write, cache/paged_cache.py:398-417. */
int ls_rope_append_fp16(const void* qkv, const void* cos, const void* sin, const int64_t* positions,
                        const int64_t* slots, void* q_out, void* k_pool, void* v_pool, void* kmin,
                        void* kmax, int batch, int q_heads, int kv_heads, int head_dim, int page,
                        int64_t max_pos, int64_t num_slots, int64_t s_qkv, int64_t s_cos, int64_t sq_b,
                        int64_t sp_t, int64_t sp_h, int64_t sb_b, int64_t sb_h, void* stream);

/* The same for the INT8 cache: rotated K into the fp16 residual (row res_idx[b]),
 * V quantised per (token, head) and scattered, bit-exact with ls_int8_decode_write;
 * with kmin / kmax (fp16 [NB, H, 128], strides sb_b, sb_h) also the page bounds of the
 * exact fp16 K, for the INT8 + sparse path.
 * Replaces `_rope_kernel` followed by `int8_decode_write`, kernels/cuda/int8_write.cu:45-78. */
int ls_rope_append_int8(const void* qkv, const void* cos, const void* sin, const int64_t* positions,
                        const int64_t* slots, const int64_t* res_idx, void* q_out, void* flat_v,
                        float* flat_v_scale, float* flat_v_zero, void* k_res, void* kmin, void* kmax,
                        int batch, int q_heads, int kv_heads, int head_dim, int64_t max_pos,
                        int64_t num_slots, int64_t num_res, int64_t s_qkv, int64_t s_cos, int64_t sq_b,
                        int64_t sb_b, int64_t sb_h, int asym, float eps, float qmax, float inv_qmax,
                        float levels, float inv_levels, float offset, void* stream);

/* Decode-step projection for a batch of m <= 32 token rows, fused with the
 * element-wise work either side of it:
 *   out[m, n] = f(x)[m, k] . w[n, k]^T (+ bias[n]),  fp16 in, fp32 accumulate, fp16 out.
 *   mode & LS_GEMM_NORM:   f(x) = RMSNorm(x (+ res)) * gamma with the fp16 rounding
 *       sequence of ls_rms_norm; with `res`, res_out <- fp16(x + res) as well
 *       (res_out must not alias x or res).
 *   mode & LS_GEMM_SWIGLU: w is [gate; up] stacked ([n, k], n = 2 I) and out is
 *       [m, I] = fp16(fp16(silu(gate)) * up) of the fp16-rounded products.
 *   mode & LS_LAUNCH_PROGRAMMATIC: the first weight loads are issued before the
 *       kernel synchronises on the previous kernel of the stream.
 *   add_res (no SWIGLU): out = fp16(fp16(product + bias) + add_res[m, n]), the residual
 *       add that follows o_proj / down_proj; with sumsq_out ([64][n / 32] floats, a
 *       row's partials contiguous) each tile also leaves the per-row sums of out^2
 *       over its 32 columns, which a later
 *       LS_GEMM_NORM call takes as sumsq_in (+ sumsq_tiles = n / 32 of THAT call, its
 *       k / 32) instead of reading whole rows for its statistics (res must then be NULL).
 * k is cut into `splits` slices across CTAs (grid = n / 32 tiles x splits; pick
 * splits so that the grid is about 2 CTAs per SM); with splits > 1 `part` must
 * hold (n / 32) * splits * 16 * ceil(m / 16) * 32 floats (k / 32 / splits <= 48 required) (n / 32 -> I / 16 tiles
 * with SWIGLU) and `counters` one int32 per tile, zeroed once before first use
 * (every launch leaves them at zero). The sum over splits is taken in split order
 * by whichever CTA finishes last, so results do not depend on timing.
 * Needs k % 32 == 0, n % 32 == 0, 16-byte aligned rows. Strides in elements.
 * In LatentServe these are the four `nn.Linear` calls of a Qwen2 decoder layer
 * (model/latentserve_qwen.py:397-451 runs them through Hugging Face modules)
 * together with `rms_norm` / `fused_add_rms_norm` / `silu_and_mul`,
 * kernels/fused_elementwise.py:194-232. */
#define LS_GEMM_NORM 1
#define LS_GEMM_SWIGLU 2
int ls_skinny_gemm(const void* x, const void* res, const void* gamma, void* res_out,
                   const float* sumsq_in, int sumsq_tiles, const void* w, const void* bias,
                   const void* add_res, float* sumsq_out, void* out, float* part, int32_t* counters,
                   int m, int n, int k, int splits, int mode, float eps, int64_t sx, int64_t sres,
                   int64_t sres_out, int64_t sw, int64_t sadd, int64_t sout, void* stream);

/* The fused QKV projection of a decode step with RoPE and the fp16 cache append in
 * its epilogue: ls_skinny_gemm (mode: LS_GEMM_NORM and the launch flags; gamma,
 * sumsq_in, part / counters, splits as there) over w [(q_heads + 2 kv_heads) * 128, k]
 * with bias, followed -- on the fp16-rounded projection output, with the roundings of
 * ls_rope_append_fp16 -- by the rotation of the q and k heads (cos, sin
 * [max_pos, 128], positions [m]) and the stores of ls_rope_append_fp16: q_out
 * [m, q_heads * 128], the rotated K row and the V row at flat slot slots[m] of the
 * pools, the page's K bounds when kmin / kmax are given. Bit-identical to
 * ls_skinny_gemm + ls_rope_append_fp16; one launch instead of two. m <= 32.
 * Replaces, in GQAAttention.forward (model/attention/gqa.py:236-267), the QKV
 * projections, `rope_qk` (kernels/fused_elementwise.py:154-182) and
 * PagedKVCache.write (cache/paged_cache.py:398-417). */
int ls_qkv_rope_append_fp16(const void* x, const void* gamma, const float* sumsq_in, int sumsq_tiles,
                            const void* w, const void* bias, const void* cos, const void* sin,
                            const int64_t* positions, const int64_t* slots, void* q_out, void* k_pool,
                            void* v_pool, void* kmin, void* kmax, float* part, int32_t* counters, int m,
                            int q_heads, int kv_heads, int head_dim, int page, int k, int splits,
                            int mode, float eps, int64_t max_pos, int64_t num_slots, int64_t sx,
                            int64_t sw, int64_t s_cos, int64_t sq_b, int64_t sp_t, int64_t sp_h,
                            int64_t sb_b, int64_t sb_h, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LATENTSERVE_B200_H */
