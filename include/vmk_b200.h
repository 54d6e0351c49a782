/* libvmk_b200: C ABI of the B200 (sm_100a) kernels for the three attention-decode ops `prefix`, `spec`
 * and `dsa`.
 *
 * The reference project has no native boundary: each op is reached through a Python module exposing
 * `def kernel(...)`, called by its verifier as fn(**inputs) (reference verify.py:35-37, 44-45, 139).
 * The entry points below are what such a kernel module binds instead of its Metal launches; each one
 * cites the reference launch path it replaces.
 *
 * Conventions for every entry point
 *   - All tensor pointers are DEVICE pointers to C-contiguous arrays; `fp16` means IEEE binary16.
 *     Inputs are borrowed and never written.  Pointers must be 16-byte aligned.
 *   - `ws` is caller-provided device scratch of at least vmk_<op>_workspace_bytes(...) bytes,
 *     256-byte aligned.  The library never allocates device memory and never synchronises; all work is
 *     enqueued on `stream` (a cudaStream_t passed as void*).  Calls on different streams are
 *     independent when their workspaces differ.
 *   - `status` (nullable) is a device int32 the kernels OR bits into when a bounded device-side wait
 *     ran out (bit 0) or an out-of-range index was clamped (bit 1).  The caller zeroes it and reads it
 *     back after synchronising.
 *   - Return value: VMK_OK or a negative VMK_E_* code; vmk_error_string() names it.  No C++
 *     exception crosses the boundary.
 */
#ifndef VMK_B200_H_
#define VMK_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define VMK_API __attribute__((visibility("default")))
#else
#define VMK_API
#endif

#define VMK_OK 0
#define VMK_E_BADARG (-1)       /* null / misaligned pointer, non-positive dimension */
#define VMK_E_UNSUPPORTED (-2)  /* shape outside what the kernels implement (see each entry point) */
#define VMK_E_WORKSPACE (-3)    /* ws_bytes smaller than vmk_<op>_workspace_bytes(...) */
#define VMK_E_LAUNCH (-4)       /* the CUDA runtime rejected a launch */
#define VMK_E_DRIVER (-5)       /* tensor-map encoding failed / driver entry point missing */
#define VMK_E_TOO_LARGE (-6)    /* the problem needs more scratch than a built-in static buffer holds */
#define VMK_E_NOMEM (-7)        /* the device had no room left for the library's static device buffers */

#define VMK_DSA_TOPK 2048
#define VMK_SPEC_MAX_DRAFTS 128

VMK_API int vmk_version(void);
VMK_API const char* vmk_error_string(int code);

/* ---- prefix: shared-prefix decode -------------------------------------------------------------
 * Replaces the two Metal launches of the reference kernel module (kernels/prefix_opus55_v8.py:282-355:
 * fused prefix-tile / suffix-stream pass, then the log-sum-exp combine).
 *   q (N,Hq,D)  kp,vp (Hkv,P,D)  ks,vs (N,Hkv,S,D)  out (N,Hq,D), all fp16.  D must be 128, Hq a
 *   multiple of Hkv with Hq/Hkv <= 16.
 *   slens (N) int32, nullable: true suffix length of each request (0..S); NULL means S for all.
 */
VMK_API size_t vmk_prefix_workspace_bytes(int N, int Hq, int Hkv, int D, int P, int S);
VMK_API int vmk_prefix_decode(const void* q, const void* kp, const void* vp, const void* ks, const void* vs,
                      const int32_t* slens, void* out, int N, int Hq, int Hkv, int D, int P, int S,
                      void* ws, size_t ws_bytes, int32_t* status, void* stream);

/* vmk_prefix_decode over a PAGED cache (the variant the reference names and leaves out, README.md:141-142; its
 * contiguous launch path is kernels/prefix_opus55_v8.py:282-355).
 *   k_pages, v_pages (pages, Hkv, page_size, D) fp16: one pool for the shared prefix and every private suffix;
 *   page_size a multiple of 64.
 *   prefix_table (prefix_pages) int32: keys [i*page_size, (i+1)*page_size) of the shared prefix live in page
 *   prefix_table[i]; prefix_pages * page_size >= P.
 *   suffix_table (N, suffix_stride) int32, slens (N) int32: request n's private suffix is slens[n] <= S keys in
 *   pages suffix_table[n][0..]; suffix_stride * page_size >= S.  Both may be null when S == 0.
 * A page id outside [0, pages) reads as zeros; rows of a page beyond the end of its prefix or suffix may hold
 * anything (NaN included).  Workspace: vmk_prefix_workspace_bytes(N, Hq, Hkv, D, P, S).  The result equals
 * vmk_prefix_decode on the de-paged tensors bit for bit.  bf16 = 0: fp16 tensors, 1: bf16 tensors. */
VMK_API int vmk_prefix_decode_paged(const void* q, const void* k_pages, const void* v_pages, int pages, int page_size,
                                    const int32_t* prefix_table, int prefix_pages, const int32_t* suffix_table,
                                    int suffix_stride, const int32_t* slens, void* out, int N, int Hq, int Hkv,
                                    int D, int P, int S, int bf16, void* ws, size_t ws_bytes, int32_t* status,
                                    void* stream);

/* ---- spec: speculative chain / tree verification ----------------------------------------------
 * Replaces the reference's permute / partial / combine launches (kernels/spec_opus55_v7.py:467-521).
 *   q (B,kd,Hq,D)  k,v (B,Hkv,L,D)  out (B,kd,Hq,D) fp16.  The drafts are the last kd cache positions.
 *   bits (B,kd,bits_words) uint32, little-endian words: bit j of row (b,i) set = draft i attends draft
 *   j.  bits_words = 1 is the reference's (B,kd) int32 layout (ops/spec.py:56); kd <= 32*bits_words,
 *   kd <= VMK_SPEC_MAX_DRAFTS, kd <= L.
 */
VMK_API size_t vmk_spec_workspace_bytes(int B, int kd, int Hq, int Hkv, int D, int L);
VMK_API int vmk_spec_verify(const void* q, const void* k, const void* v, const uint32_t* bits, int bits_words,
                    void* out, int B, int kd, int Hq, int Hkv, int D, int L, void* ws, size_t ws_bytes,
                    int32_t* status, void* stream);

/* vmk_spec_verify over a PAGED cache, the layout serving stacks keep (the reference names the paged variant as
 * the one it left out, README.md:141-142; its contiguous launch path is kernels/spec_opus55_v7.py:467-521).
 *   k_pages, v_pages (pages, Hkv, page_size, D) fp16: one pool for all requests; page_size a multiple of 64.
 *   page_table (B, table_stride) int32: keys [i*page_size, (i+1)*page_size) of request b live in page
 *   page_table[b][i]; table_stride * page_size >= L.  Entries beyond ceil(L / page_size) are not read; a page id
 *   outside [0, pages) reads as zeros.  Rows of the last page beyond L may hold anything (NaN included).
 * Everything else as vmk_spec_verify, same workspace size; the result equals vmk_spec_verify on the
 * de-paged cache bit for bit.  bf16 = 0: fp16 tensors, 1: bf16 tensors. */
VMK_API int vmk_spec_verify_paged(const void* q, const void* k_pages, const void* v_pages, const int32_t* page_table,
                                  int pages, int page_size, int table_stride, const uint32_t* bits, int bits_words,
                                  void* out, int B, int kd, int Hq, int Hkv, int D, int L, int bf16, void* ws,
                                  size_t ws_bytes, int32_t* status, void* stream);

/* vmk_spec_verify without any caller-provided scratch.  This entry point has no counterpart in the
 * reference; it exists for hosts that may not allocate device memory around the call: a serving runtime
 * that hands every byte of HBM to its own pools at start-up and loads this library as a plug-in with no
 * allocator to call back into, or a latency-critical loop whose rules forbid cudaMalloc once it is
 * running.  The split partials live in a static device array inside the library image
 * (VMK_SPEC_NOALLOC_SCRATCH_BYTES on every GPU that loads the library, held until the process exits),
 * so there is neither `ws` nor `ws_bytes`; inputs and output are still the caller's.
 *   - A shape whose partials would not fit is refused with VMK_E_TOO_LARGE before anything is launched;
 *     vmk_spec_workspace_bytes(...) <= VMK_SPEC_NOALLOC_SCRATCH_BYTES tells in advance.
 *   - The array becomes resident when the CUDA module that holds it is loaded on a device, which under the
 *     runtime's default lazy loading is the first use of a kernel or symbol of that module -- typically the
 *     first call of this entry point, not the loading of the library.  A host that claims all remaining
 *     device memory for its own pools must therefore make one warm-up call on each device BEFORE it does so
 *     (or run with CUDA_MODULE_LOADING=EAGER, which reserves the bytes when the library's context is set up);
 *     otherwise that first call can fail with VMK_E_NOMEM, or take the bytes out of memory the host thinks it
 *     owns.
 *   - The first call on each device also looks up the array's device address (cudaGetSymbolAddress); make
 *     that first call before any stream capture begins on that device.
 *   - All calls on a device share the one array and it keeps the previous call's contents.  Nothing in
 *     it needs clearing, but calls whose kernels overlap on the GPU (different streams) race on it:
 *     serialise them, or use vmk_spec_verify with separate workspaces.
 *   - It performs no cudaMalloc / cudaFree and calls no allocating library routine. */
#define VMK_SPEC_NOALLOC_SCRATCH_BYTES (32u << 20)
VMK_API int vmk_spec_verify_noalloc(const void* q, const void* k, const void* v, const uint32_t* bits,
                                    int bits_words, void* out, int B, int kd, int Hq, int Hkv, int D, int L,
                                    int32_t* status, void* stream);

/* ---- dsa: DeepSeek sparse attention decode ----------------------------------------------------
 * Replaces the reference's indexer / select / gather+QK / softmax / PV / reduce launches
 * (kernels/dsa_opus55_v7.py:946-977).  Fixed head geometry (ops/dsa.py:15): 128 heads, rows of
 * 576 = 512 latent + 64 rope, 64 indexer heads of width 128, top-2048.
 *   q (B,128,576)  kv (B,L,576)  iq (B,64,128)  ik (B,L,128) fp16;  w (B,64) fp32;
 *   lens (B) int32, nullable: valid cache length per request (1..L);  out (B,128,512) fp16.
 *   idx_out (B,2048) int32 and cnt_out (B) int32, nullable: the selected positions (ascending) and how
 *   many are valid, exposed so the integer stage can be checked bit for bit.
 * vmk_dsa_decode runs the three stages below back to back; they are also exported one by one.
 */
VMK_API size_t vmk_dsa_workspace_bytes(int B, int L);
VMK_API int vmk_dsa_decode(const void* q, const void* kv, const void* iq, const void* ik, const float* w,
                   const int32_t* lens, void* out, int32_t* idx_out, int32_t* cnt_out, int B, int L,
                   void* ws, size_t ws_bytes, int32_t* status, void* stream);

/* Stage 1 (kernels/dsa_opus55_v7.py:629-661): scores (B,L) fp32 = sum_h w[h]*relu(iq[h].ik[l]), fp32
 * accumulation.  Positions at or beyond lens[b] are left unwritten. */
VMK_API int vmk_dsa_indexer(const void* iq, const void* ik, const float* w, const int32_t* lens, float* scores,
                    int B, int L, int32_t* status, void* stream);
/* Stage 2 (kernels/dsa_opus55_v7.py:100-307): exact top-2048 of scores[b,:n], n = lens[b] or L; all n
 * positions when n <= 2048.  Ties at the boundary go to the lowest positions; NaN scores rank last.
 * idx (B,2048) ascending, entries beyond cnt[b] are 0. */
VMK_API int vmk_dsa_select(const float* scores, const int32_t* lens, int32_t* idx, int32_t* cnt, int B, int L,
                   void* stream);
/* Stages 1 and 2 with the first level of the select fused into the indexer, as vmk_dsa_decode runs them
 * (the reference fuses a histogram of the top key bits into its indexer the same way,
 * kernels/dsa_opus55_v7.py:629-661, and its select starts from it, 124-150).  hist (B,2048) uint32 is
 * zeroed and then filled by vmk_dsa_indexer_hist: hist[b][k] counts the valid positions of request b whose
 * score key has k as its top 11 bits (key = order-preserving map of the fp32 score, NaN -> 0, -0 = +0). */
VMK_API int vmk_dsa_indexer_hist(const void* iq, const void* ik, const float* w, const int32_t* lens,
                                 float* scores, uint32_t* hist, int B, int L, int32_t* status, void* stream);
VMK_API int vmk_dsa_select_hist(const float* scores, const uint32_t* hist, const int32_t* lens, int32_t* idx,
                                int32_t* cnt, int B, int L, void* stream);
/* Compaction of the selected rows (the reference's dsa_gather_v7, kernels/dsa_opus55_v7.py:537-550, 744-746,
 * 853): kv_sel (B,2048,576) fp16 receives row idx[b][j] of request b at position j for j < cnt[b]; idx_sel
 * (B,2048) receives j, so that vmk_dsa_attend(q, kv_sel, idx_sel, cnt, out, B, 2048, ...) equals
 * vmk_dsa_attend(q, kv, idx, cnt, out, B, L, ...) bit for bit.  kv only has to be readable from the device: it
 * may be page-locked host memory, and a host-resident cache then sends 2048 rows per request over the link
 * instead of L.  kv_sel and idx_sel are device memory; rows at or beyond cnt[b] are left untouched. */
VMK_API int vmk_dsa_gather(const void* kv, const int32_t* idx, const int32_t* cnt, void* kv_sel, int32_t* idx_sel,
                           int B, int L, int32_t* status, void* stream);
/* Stage 3 (kernels/dsa_opus55_v7.py:839-871): absorbed-MLA attention over the selected rows. */
VMK_API size_t vmk_dsa_attend_workspace_bytes(int B);
VMK_API int vmk_dsa_attend(const void* q, const void* kv, const int32_t* idx, const int32_t* cnt, void* out,
                   int B, int L, void* ws, size_t ws_bytes, int32_t* status, void* stream);

/* ---- batch invariance --------------------------------------------------------------------------------
 * The fourth layer of the reference's judge, which its public verify.py leaves out (ONE-PAGER.md:15,24-25): a row
 * computed in a batch must have the same bits as the same row computed alone.  The default planners choose
 * kernels, layouts and cut points for the batch at hand, which changes the order of some fp32 sums; with
 * vmk_set_batch_invariant(1) they are fixed (warp-level attention kernel, 2048-key splits, four parts per dsa
 * unit) and every op of this library holds the property, at a lower speed.  Process-wide; returns VMK_OK. */
VMK_API int vmk_set_batch_invariant(int on);

/* ---- decode: plain single-token decode --------------------------------------------------------------
 * The op the reference measures beside its three ("single-token decode", POST.md:42,47) and names as the natural
 * fourth on the same main loop; it ships no kernel for it.  One query per request over that request's own cache:
 *   q (B,Hq,D)  k,v (B,Hkv,L,D)  lens (B) int32, 1 <= lens[b] <= L  out (B,Hq,D); bf16 = 0 (fp16) or 1.
 * Rows [lens[b], L) of request b may hold anything (NaN included).  The paged form takes one pool
 * (pages,Hkv,page_size,D) and page_table (B,table_stride) as vmk_spec_verify_paged does, L then being the
 * largest length (table_stride * page_size >= L). */
VMK_API size_t vmk_decode_workspace_bytes(int B, int Hq, int Hkv, int D, int L);
VMK_API int vmk_decode(const void* q, const void* k, const void* v, const int32_t* lens, void* out, int B, int Hq,
                       int Hkv, int D, int L, int bf16, void* ws, size_t ws_bytes, int32_t* status, void* stream);
VMK_API int vmk_decode_paged(const void* q, const void* k_pages, const void* v_pages, const int32_t* page_table,
                             int pages, int page_size, int table_stride, const int32_t* lens, void* out, int B,
                             int Hq, int Hkv, int D, int L, int bf16, void* ws, size_t ws_bytes, int32_t* status,
                             void* stream);

/* ---- prefix and spec on bf16 tensors ---------------------------------------------------------------
 * vmk_prefix_decode (kernels/prefix_opus55_v8.py:282-355) and vmk_spec_verify (kernels/spec_opus55_v7.py:467-521)
 * with q, K, V and out in bf16; the reference's kernels are fp16 only (README.md:140).  Same shapes, workspaces,
 * masks and status word; scores, statistics and accumulators stay fp32, P is rounded to bf16 before P.V. */
VMK_API int vmk_prefix_decode_bf16(const void* q, const void* kp, const void* vp, const void* ks, const void* vs,
                                   const int32_t* slens, void* out, int N, int Hq, int Hkv, int D, int P, int S,
                                   void* ws, size_t ws_bytes, int32_t* status, void* stream);
VMK_API int vmk_spec_verify_bf16(const void* q, const void* k, const void* v, const uint32_t* bits, int bits_words,
                                 void* out, int B, int kd, int Hq, int Hkv, int D, int L, void* ws, size_t ws_bytes,
                                 int32_t* status, void* stream);

/* ---- dsa on bf16 tensors --------------------------------------------------------------------------
 * The reference's kernels read fp16 only and produce invalid values on bf16 inputs (README.md:140); these are
 * vmk_dsa_decode (kernels/dsa_opus55_v7.py:946-977), vmk_dsa_indexer_hist and vmk_dsa_attend with q, kv, iq,
 * ik and out in bf16 (w stays fp32, scores fp32, indices int32; vmk_dsa_select_hist and vmk_dsa_gather do not
 * depend on the 16-bit type).  Same shapes, workspaces and status word.  Products of bf16 values are exact in
 * fp32 as those of fp16 values are; P is rounded to bf16 before P.V and the output to bf16. */
VMK_API int vmk_dsa_decode_bf16(const void* q, const void* kv, const void* iq, const void* ik, const float* w,
                                const int32_t* lens, void* out, int32_t* idx_out, int32_t* cnt_out, int B, int L,
                                void* ws, size_t ws_bytes, int32_t* status, void* stream);
VMK_API int vmk_dsa_indexer_hist_bf16(const void* iq, const void* ik, const float* w, const int32_t* lens,
                                      float* scores, uint32_t* hist, int B, int L, int32_t* status, void* stream);
VMK_API int vmk_dsa_attend_bf16(const void* q, const void* kv, const int32_t* idx, const int32_t* cnt, void* out,
                                int B, int L, void* ws, size_t ws_bytes, int32_t* status, void* stream);

/* vmk_dsa_decode over a PAGED cache (the layout of serving stacks; the reference names the paged variant as
 * left out, README.md:141-142; its contiguous launch path is kernels/dsa_opus55_v7.py:946-977).
 *   kv_pages (pages, page_size, 576), ik_pages (pages, page_size, 128): one pool each, paged alike; page_size a
 *   multiple of 128.  page_table (B, table_stride) int32: positions [i*page_size, (i+1)*page_size) of request b
 *   are page page_table[b][i] of both pools.  lens (B) is required; L is the largest length the call may see
 *   (2048 < L <= table_stride * page_size) and sizes the workspace: vmk_dsa_workspace_bytes(B, L).
 * Positions at or beyond lens[b] may hold anything.  idx_out holds logical positions.  bf16 = 0 / 1.  The result
 * equals vmk_dsa_decode on the de-paged tensors bit for bit. */
VMK_API int vmk_dsa_decode_paged(const void* q, const void* kv_pages, const void* iq, const void* ik_pages,
                                 const float* w, const int32_t* page_table, int pages, int page_size,
                                 int table_stride, const int32_t* lens, void* out, int32_t* idx_out, int32_t* cnt_out,
                                 int B, int L, int bf16, void* ws, size_t ws_bytes, int32_t* status, void* stream);

/* Stage 1 with the index queries and keys stored in fp8, the format DeepSeek-V3.2-style deployments keep their
 * index keys in; the reference's op takes fp16 (ops/dsa.py:22-50) and lists this step as outside it
 * (ops/dsa.py:8-9).  It halves the stream that dominates the op.
 *   iq8 (B,64,128), ik8 (B,L,128): e4m3 bytes;  iq_scale (B,64), ik_scale (B,L) fp32, positive: the value of an
 *   element is scale * e4m3.  scores[b,l] = ik_scale[b,l] * sum_h w[b,h] * iq_scale[b,h] * relu(iq8[b,h] . ik8[b,l])
 *   (the scales are positive, so they commute with the ReLU); hist as vmk_dsa_indexer_hist.
 * Continue with vmk_dsa_select_hist and vmk_dsa_attend. */
VMK_API int vmk_dsa_indexer_hist_fp8(const void* iq8, const float* iq_scale, const void* ik8, const float* ik_scale,
                                     const float* w, const int32_t* lens, float* scores, uint32_t* hist, int B, int L,
                                     int32_t* status, void* stream);

/* The step before stage 1: the projection that produces the indexer's queries and head weights, which the
 * reference keeps outside its op (ops/dsa.py:8-9 names the projections that produce q / iq / w as not part of it;
 * there is no reference kernel or truth for it: the float64 statement lives in oracle/ref64.py).
 *   x (B, Dx) activation; wq (8192, Dx), ww (64, Dx): weights stored (out features, in features) as a linear layer
 *   keeps them; all three fp16 (bf16 = 0) or bf16 (1); Dx a multiple of 8.
 *   iq_out (B, 64, 128), same 16-bit type: iq[b, h, d] = sum_k x[b, k] * wq[h * 128 + d, k], fp32 accumulation,
 *   rounded once.  w_out (B, 64) fp32: w[b, h] = w_scale * sum_k x[b, k] * ww[h, k].
 * Both outputs are what vmk_dsa_decode / vmk_dsa_indexer_hist take as iq and w.  Positional encodings, if the model
 * applies any to its index queries, are the caller's to apply between the two calls. */
VMK_API int vmk_dsa_index_project(const void* x, const void* wq, const void* ww, float w_scale, void* iq_out,
                                  float* w_out, int B, int Dx, int bf16, int32_t* status, void* stream);

/* ---- merge of split partials -------------------------------------------------------------------
 * Log-sum-exp merge used after a KV split across GPUs (the reference merges its in-GPU splits the
 * same way, kernels/prefix_opus55_v8.py:211-261).  m, l (parts,rows) and o (parts,rows,D) fp32 with m
 * in the base-2 scaled-score domain the partial kernels emit; out (rows,D) fp16. */
VMK_API int vmk_lse_merge(const float* m, const float* l, const float* o, int parts, int rows, int D, void* out,
                  void* stream);

/* Split partials of one rank, for the multi-GPU KV split: the same computations as vmk_prefix_decode /
 * vmk_spec_verify restricted to keys [key_lo, key_hi) of the shared prefix / the cache, returning the
 * un-normalised partial (m, l, o) per output row instead of the final output.
 *   part_m, part_l (rows) fp32, part_o (rows, D) fp32 with rows = N*Hq (prefix) or B*kd*Hq (spec). */
VMK_API int vmk_prefix_partial(const void* q, const void* kp, const void* vp, const void* ks, const void* vs,
                       const int32_t* slens, int N, int Hq, int Hkv, int D, int P, int S, int key_lo,
                       int key_hi, int with_suffix, float* part_m, float* part_l, float* part_o, void* ws,
                       size_t ws_bytes, int32_t* status, void* stream);
VMK_API int vmk_spec_partial(const void* q, const void* k, const void* v, const uint32_t* bits, int bits_words,
                     int B, int kd, int Hq, int Hkv, int D, int L, int key_lo, int key_hi, float* part_m,
                     float* part_l, float* part_o, void* ws, size_t ws_bytes, int32_t* status, void* stream);

/* The same partials as ONE packed record per output row, `records` (rows, 130) fp32 = (m, l, o[128]): the form
 * in which a rank's partials cross to another GPU in a single exchange (one all-to-all or all-gather of one
 * buffer), and the input of vmk_lse_merge_packed.  The reference merges its in-GPU splits from separate
 * (m, l) and o arrays (kernels/prefix_opus55_v8.py:211-261); its split plan is kernels/prefix_opus55_v8.py:320-331.
 *   vmk_prefix_partial_packed: q points at head h0 of request 0 of a (N, q_heads, D) tensor and the call covers
 *   heads [h0, h0 + Hq) (q_heads >= Hq; q_heads == Hq for all heads), with kp, vp (Hkv, P, D) and ks, vs
 *   (N, Hkv, S, D) the matching slice of kv heads.  rows = N*Hq, row (n, head) at n*Hq + head.  key_lo == key_hi
 *   skips the shared prefix (suffix-only partials); with_suffix = 0 skips the private suffixes; at least one of
 *   the two must be left.  bf16 = 0 / 1.  Workspace: vmk_prefix_workspace_bytes(N, Hq, Hkv, D, P, S).
 *   vmk_spec_partial_packed: as vmk_spec_partial; rows = B*kd*Hq.  mask_start is the first position of k, v that
 *   is a draft: -1 (or L - kd) when the tensor ends with the drafts; any value >= L when k, v are a slice of a
 *   longer cache whose drafts lie in another rank's slice, so that no key of this call is masked.
 *   vmk_lse_merge_packed: records (parts, rows, 130) -> out (rows, 128) fp16 (bf16 = 0) or bf16 (1); D must be 128. */
VMK_API int vmk_prefix_partial_packed(const void* q, int q_heads, const void* kp, const void* vp, const void* ks,
                                      const void* vs, const int32_t* slens, int N, int Hq, int Hkv, int D, int P,
                                      int S, int key_lo, int key_hi, int with_suffix, int bf16, float* records,
                                      void* ws, size_t ws_bytes, int32_t* status, void* stream);
VMK_API int vmk_spec_partial_packed(const void* q, const void* k, const void* v, const uint32_t* bits, int bits_words,
                                    int B, int kd, int Hq, int Hkv, int D, int L, int key_lo, int key_hi,
                                    int mask_start, int bf16, float* records, void* ws, size_t ws_bytes,
                                    int32_t* status, void* stream);
VMK_API int vmk_lse_merge_packed(const float* records, int parts, int rows, int D, int bf16, void* out, void* stream);

/* ---- process-wide behaviour switches, for A/B comparisons and cross-checks ----------------------------
 * No counterpart in the reference (its variants are separate kernel files).  Each returns VMK_OK.
 *   vmk_attn_set_tc(0): prefix / spec row tiles of more than 64 rows use the warp-level kernel instead of
 *   the tcgen05 one (1, the default).
 *   vmk_dsa_set_indexer_variant(v), vmk_dsa_set_attend_variant(v): 1 = tcgen05 kernels (the indexer's default),
 *   0 = the warp-level mma.sync kernels kept as cross-checks (fp16, contiguous caches only).  The attend stage
 *   also takes 2 = the tcgen05 kernel of 1 with its rows gathered by TMA (tile::gather4) instead of cp.async (the
 *   result has the same bits) and 3 = the tcgen05 kernel that gives a request to a cluster of two CTAs which
 *   share the score product (its default).  Other values are refused. */
VMK_API int vmk_attn_set_tc(int on);
/*   vmk_prefix_set_side_by_side(0): a prefix call with 512 or more private suffixes (requests x kv heads) and more
 *   than 64 stacked rows runs its tensor-bound prefix kernel and its HBM-bound suffix kernel one after the other on the caller's
 *   stream, instead of side by side (1, the default: the prefix kernel takes one wave on two thirds of the SMs and
 *   the suffix kernel runs on a second stream the library creates per device, forked from and joined to the
 *   caller's stream by events; the results have the same bits unless the prefix is cut into a different number
 *   of splits). */
VMK_API int vmk_prefix_set_side_by_side(int on);
VMK_API int vmk_dsa_set_indexer_variant(int variant);
VMK_API int vmk_dsa_set_attend_variant(int variant);
/*   vmk_dsa_set_select_cluster(c): CTAs per request of the top-k selection on rows of 32768 positions and more
 *   (1, 2, 4 or 8: that many SMs read a row together and exchange histograms through distributed shared memory);
 *   0, the default, takes the largest size whose CTAs fit in one wave.  The selection is the same set. */
VMK_API int vmk_dsa_set_select_cluster(int csize);

#ifdef __cplusplus
}
#endif
#endif /* VMK_B200_H_ */
