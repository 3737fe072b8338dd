/*
 * C ABI of the B200 (sm_100a) Qwen3-0.6B greedy-decode engine.
 *
 * The first four entry points have exactly the signatures the reference's torch
 * binding declares and calls (Tools/megakernel/qwen_ops.cpp:9-39), so that file
 * links against this library unchanged.  The qmk_* entry points are additions
 * (status codes, configuration, diagnostics) with no counterpart in the
 * reference.
 *
 * Conventions: all weight/cache/scratch pointers are DEVICE pointers owned by
 * the caller; `token_ids` of launch_ldg_prefill is a HOST pointer; every call
 * acts on the CUDA device that is current on the calling thread and on the
 * stream passed in.  The library keeps a small per-device scratch area of its
 * own (inter-CTA exchange words + status), allocated on first use.
 * The library is not re-entrant per device: one call at a time per GPU, as in
 * the reference (process-global launcher state, megakernel_5090.cu:722-742).
 */
#ifndef QWEN_MEGAKERNEL_H_
#define QWEN_MEGAKERNEL_H_

#include <cuda_runtime_api.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Per-layer weight pointer record: 12 x 8 bytes, 16-byte aligned.  Same field
 * order and size as the reference's struct (megakernel_5090.cu:91-104) and as
 * the int64 table packed by Model/Qwen06B_architecture.py:166-185.
 * All matrices are fp16 row-major [out, in]. */
struct LDGLayerWeight;

/* One decode step; the greedy token is written to *output_token_id (device).
 * Does not synchronise.  Replaces megakernel_5090.cu:1175-1218
 * (declared at qwen_ops.cpp:9-17). */
void launch_ldg_decode_direct(
    int input_token_id, int *output_token_id, const void *embed_weight,
    const struct LDGLayerWeight *layer_weights, const void *final_norm_weight,
    const void *lm_head_weight, const void *cos_table, const void *sin_table,
    void *k_cache, void *v_cache, void *hidden_buffer, void *g_activations,
    void *g_residual, void *g_q, void *g_k, void *g_v, void *g_attn_out,
    void *g_mlp_intermediate, void *g_normalized, void *block_max_vals,
    void *block_max_idxs, int num_layers, int position, int max_seq_len,
    float attn_scale, cudaStream_t stream);

/* Same contract as launch_ldg_decode_direct.  Replaces
 * megakernel_5090.cu:1220-1272 (exported there, not bound by qwen_ops.cpp). */
void launch_ldg_decode_persistent(
    int input_token_id, int *output_token_id, const void *embed_weight,
    const struct LDGLayerWeight *layer_weights, const void *final_norm_weight,
    const void *lm_head_weight, const void *cos_table, const void *sin_table,
    void *k_cache, void *v_cache, void *hidden_buffer, void *g_activations,
    void *g_residual, void *g_q, void *g_k, void *g_v, void *g_attn_out,
    void *g_mlp_intermediate, void *g_normalized, void *block_max_vals,
    void *block_max_idxs, int num_layers, int position, int max_seq_len,
    float attn_scale, cudaStream_t stream);

/* num_steps greedy tokens from first_token_id at start_position; token i is
 * written to output_log[i]; the EOS token is logged and ends the run; entries
 * after it are left untouched.  Blocks until the stream is idle.  Replaces
 * megakernel_5090.cu:1357-1436 (declared at qwen_ops.cpp:19-29). */
void launch_ldg_generate_nosync(
    int first_token_id, int num_steps, const void *embed_weight,
    const struct LDGLayerWeight *layer_weights, const void *final_norm_weight,
    const void *lm_head_weight, const void *cos_table, const void *sin_table,
    void *k_cache, void *v_cache, void *hidden_buffer, void *g_activations,
    void *g_residual, void *g_q, void *g_k, void *g_v, void *g_attn_out,
    void *g_mlp_intermediate, void *g_normalized, void *block_max_vals,
    void *block_max_idxs, int *output_log, int num_layers, int start_position,
    int max_seq_len, float attn_scale, int eos_token_id, cudaStream_t stream);

/* Fills the KV cache for num_tokens prompt tokens (HOST int32 array) at
 * positions start_position .. start_position+num_tokens-1; no LM head.
 * Blocks until done.  Replaces megakernel_5090.cu:1276-1355
 * (declared at qwen_ops.cpp:31-39). */
void launch_ldg_prefill(
    const int *token_ids, int num_tokens, const void *embed_weight,
    const struct LDGLayerWeight *layer_weights, const void *final_norm_weight,
    const void *lm_head_weight, const void *cos_table, const void *sin_table,
    void *k_cache, void *v_cache, void *hidden_buffer, void *g_activations,
    void *g_residual, void *g_q, void *g_k, void *g_v, void *g_attn_out,
    void *g_mlp_intermediate, void *g_normalized, void *block_max_vals,
    void *block_max_idxs, int num_layers, int start_position, int max_seq_len,
    float attn_scale, cudaStream_t stream);

/* ---- additions (no counterpart in the reference) ------------------------- */

/* Status codes returned by qmk_* and kept by the void entry points above. */
enum {
  QMK_OK = 0,
  QMK_ERR_CUDA = 1,          /* a CUDA runtime call failed (see qmk_last_error) */
  QMK_ERR_BAD_ARGUMENT = 2,  /* null/misaligned pointer, bad sizes */
  QMK_ERR_POSITION = 3,      /* start_position + steps exceeds max_seq_len */
  QMK_ERR_WAIT_TIMEOUT = 4,  /* a bounded device-side wait ran out */
  QMK_ERR_BAD_TOKEN = 5,     /* token id outside [0, vocab) reached the kernel */
  QMK_ERR_NOT_RESIDENT = 6   /* the persistent grid cannot be co-resident */
};

/* Layout version of LDGLayerWeight / the op surface; equals the reference's
 * abi_version() (qwen_ops.cpp:42-44). */
int qmk_abi_version(void);

/* Engine options for the current device; pass a negative value to keep one.
 *  vocab_size       rows of the tied LM head (default 151936, the reference's
 *                   compile-time LDG_VOCAB_SIZE, megakernel_5090.cu:85)
 *  rope_from_table  1: rotate with the caller's fp16 cos/sin tables as the
 *                   reference does (megakernel_5090.cu:351-352); 0 (default):
 *                   fp32 angles position * inv_freq computed in the kernel, valid
 *                   for any position
 *  split_len        target KV positions per attention work item (default 128)
 *  max_ctas         cap on the persistent grid (default: one CTA per SM)
 *  timeout_ms       budget of every device-side wait (default 2000) */
int qmk_configure(int vocab_size, int rope_from_table, int split_len, int max_ctas, int timeout_ms);

/* 64 fp32 inverse frequencies theta^(-2i/128) used when rope_from_table == 0
 * (HOST pointer).  Default: theta = 1e6. */
int qmk_set_inv_freq(const float *inv_freq64);

/* ---- engine handles ---------------------------------------------------------
 * The options above (qmk_configure, qmk_set_inv_freq, qmk_set_weight_format,
 * qmk_set_fused) are state of the library per device: two clients of one GPU
 * that differ in them would have to re-apply theirs before every op.  A handle
 * keeps one client's options and applies them together with the op under one
 * hold of the library's lock, so clients with different vocabularies, weight
 * formats or RoPE settings can share a GPU, also from several threads.  The
 * reference has no such object (its ops are free functions over one implicit
 * GPU state, qwen_ops.cpp:262-270); qmk_engine_decode / _generate / _prefill
 * take the handle first and then exactly the arguments of qmk_decode /
 * qmk_generate / qmk_prefill.  A handle call makes the handle's device the
 * calling thread's current device; the stream must belong to it. */
typedef struct qmk_engine qmk_engine;
typedef struct qmk_engine_config {
  int device;              /* CUDA device ordinal */
  int vocab_size;          /* LM-head rows; <= 0: 151936 */
  int weight_format;       /* 0 fp16, 1 FP8-E4M3 rows (see qmk_set_weight_format) */
  int rope_from_table;     /* see qmk_configure */
  int split_len;           /* <= 0: qmk_configure's value */
  int max_ctas;            /* <= 0: qmk_configure's value */
  int timeout_ms;          /* <= 0: qmk_configure's value */
  int fused;               /* 2, 1, 0 as qmk_set_fused; negative: whatever qmk_set_fused last chose */
  const float *inv_freq64; /* HOST, 64 floats, copied by qmk_engine_create; NULL: theta = 1e6 */
} qmk_engine_config;
int qmk_engine_create(const qmk_engine_config *config, qmk_engine **out);
/* Frees the handle and the K-major weight copies made for the layer tables it decoded with. */
int qmk_engine_destroy(qmk_engine *engine);
/* Makes the handle's options the device's current ones (for the entry points that take no handle). */
int qmk_engine_apply(qmk_engine *engine);
int qmk_engine_decode(
    qmk_engine *engine, int input_token_id, int *output_token_id, const void *embed_weight,
    const struct LDGLayerWeight *layer_weights, const void *final_norm_weight,
    const void *lm_head_weight, const void *cos_table, const void *sin_table,
    void *k_cache, void *v_cache, void *hidden_buffer, void *g_normalized,
    void *block_max_vals, void *block_max_idxs, int num_layers, int position,
    int max_seq_len, float attn_scale, cudaStream_t stream);
int qmk_engine_generate(
    qmk_engine *engine, int first_token_id, int num_steps, const void *embed_weight,
    const struct LDGLayerWeight *layer_weights, const void *final_norm_weight,
    const void *lm_head_weight, const void *cos_table, const void *sin_table,
    void *k_cache, void *v_cache, void *hidden_buffer, void *g_normalized,
    void *block_max_vals, void *block_max_idxs, int *output_log, int num_layers,
    int start_position, int max_seq_len, float attn_scale, int eos_token_id,
    int synchronize, cudaStream_t stream);
int qmk_engine_prefill(
    qmk_engine *engine, const int *token_ids_host, int num_tokens, const void *embed_weight,
    const struct LDGLayerWeight *layer_weights, const void *final_norm_weight,
    const void *cos_table, const void *sin_table, void *k_cache, void *v_cache,
    int num_layers, int start_position, int max_seq_len, float attn_scale,
    cudaStream_t stream);

/* Debug: when non-null, decode steps also write every logit to
 * logits_out[step * vocab_size + row] (DEVICE fp32).  Null switches it off. */
int qmk_set_logits_dump(float *logits_out);

/* Weight format of ALL matrices reached through the layer table, the embedding
 * and the LM head (norm vectors stay fp16).  0 (default): fp16 row-major [out,in].
 * 1: FP8-E4M3 rows - each row is `in` e4m3 bytes followed by a 16-byte trailer
 * whose first 4 bytes are the row's fp32 scale (w = scale * e4m3); row stride
 * in + 16 bytes.  Activations, accumulation and the KV cache are unchanged.
 * 2: NVFP4 rows - `in`/2 bytes of e2m1 pairs (element 2i in the low nibble of byte i), `in`/16 e4m3 scales (one per
 * 16 values), then a 16-byte trailer whose first 4 bytes are the matrix's fp32 tensor scale
 * (w = tensor_scale * block_scale * e2m1); row stride in/2 + in/16 + 16 bytes.  Format 2 is read by the tensor-core
 * entry points only (qmk_prefill_chunked, qmk_decode_batched, qmk_gemm_packed_tn); the persistent kernels refuse it. */
int qmk_set_weight_format(int format);

/* Performance knobs; negative keeps a value.  spin_sleep_ns: nanosleep between
 * polls of an exchange word (default: 600 for the unfused kernel, 0 for the fused one; setting it sets both).  l2_evict_first: 1 (default) streams
 * weights with an evict-first L2 policy, 0 uses the default policy. */
int qmk_set_tuning(int spin_sleep_ns, int l2_evict_first);
/* More knobs; negative keeps a value.  repl (1, 2 or 4): copies of the exchange
 * area; producers publish every word to all copies and CTA i polls copy i % repl,
 * which divides the number of pollers per cache line (default 4).  stream_inflight: cap on
 * weight/KV chunks in flight per SM during the layer phases (0 = ring depth). */
int qmk_set_tuning2(int repl, int stream_inflight);

/* Chunked prefill (qmk_prefill_chunked): 1 (default) runs the causal attention on the tcgen05 tensor cores (S and O
 * accumulators in TMEM, K / V tiles by TMA from the cache), 0 on the mma.sync kernel.  Same tolerance against the
 * oracle either way; negative keeps. */
int qmk_set_prefill_attention(int tensor_core);

/* Batched decode (qmk_decode_batched): 1 (default) runs the per-sequence attention on mma.sync tensor-core tiles (cache
 * rows by tiled TMA through per-sequence descriptors the call encodes), 0 on the CUDA-core kernel it replaces.  Same
 * tolerance against the oracle either way; negative keeps. */
int qmk_set_decode_attention(int tensor_core);

/* Batched decode (qmk_decode_batched): 1 (default) launches the ~200 kernels of a decode step as programmatic
 * dependents of one another - each kernel is scheduled while its predecessor still runs, sets itself up, streams the
 * operands no kernel of the step writes (weight tiles, cache rows of earlier steps) and only then waits for the
 * predecessor to complete; 0 launches them strictly one after the other.  The same switch covers the GEMMs of
 * qmk_prefill_chunked / qmk_prefill_packed (only the GEMMs: the other kernels of a prefill pass always launch
 * plainly).  Same results either way; negative keeps. */
int qmk_set_step_overlap(int enabled);

/* Kernel choice for one sequence (qmk_decode / qmk_generate / qmk_prefill); negative keeps a value.
 *  fused  2 (default) or 1: the fused kernel - the O and down projections run as split-K slices on the CTAs that
 *         produced their inputs, and the two residual sums of a layer are all-reduced in 64-bit integer
 *         accumulators (four cross-CTA hand-overs per layer).  It reads K-major copies of W_o and W_down that
 *         the library makes from the caller's matrices (294 MB for 28 fp16 layers) on the first call with a
 *         layer table and re-checks by sampled hashes on every call.  Grids below 74 CTAs and
 *         qmk_generate_static use the unfused kernel (six hand-overs, no copies).  0: always unfused.
 *         2 multiplies weight rows on the tensor cores (mma.sync tiles of 16 rows, the fp32 activation vector
 *         split into two fp16 columns); it needs fp16 weights and a vocabulary that is a multiple of 4, and falls
 *         back to 1 (CUDA-core row products, any format) otherwise.
 *  red_copies  1 or 2 accumulator copies per sum (2 halves the same-address add queue, doubles the words read).
 * The reference has neither (its layer is eight grid barriers, megakernel_5090.cu:879-915). */
int qmk_set_fused(int fused, int red_copies);
/* Marks every K-major copy on the current device stale: the next call rebuilds it.  Needed only after editing
 * W_o / W_down in place in a way the sampled hashes may miss. */
int qmk_invalidate_weights(void);
/* Frees the K-major copies made for this layer table (null: all tables) on the current device. */
int qmk_release_weights(const struct LDGLayerWeight *layer_weights);

/* Debug: when non-null, every CTA writes globaltimer stamps (ns) of the phase
 * boundaries of the LAST step of each launch to timestamps[cta * 768 + slot]
 * (DEVICE, >= grid * 768 words): slot layer*12 + k, k = 0 layer start, 1 QKV done,
 * 2 attention done, 3 merge done, 4 attention output received, 5 O-proj done,
 * 6 residual received, 7 gate/up done, 8 MLP activations received, 9 down-proj
 * done, 10 layer output received; slots num_layers*12 + {0,1,2}: LM head start,
 * LM head rows done, next token known.  Null switches it off. */
int qmk_set_profile_buffer(unsigned long long *timestamps);

/* Status-returning twins of the three void launchers. */
int qmk_decode(
    int input_token_id, int *output_token_id, const void *embed_weight,
    const struct LDGLayerWeight *layer_weights, const void *final_norm_weight,
    const void *lm_head_weight, const void *cos_table, const void *sin_table,
    void *k_cache, void *v_cache, void *hidden_buffer, void *g_normalized,
    void *block_max_vals, void *block_max_idxs, int num_layers, int position,
    int max_seq_len, float attn_scale, cudaStream_t stream);
int qmk_generate(
    int first_token_id, int num_steps, const void *embed_weight,
    const struct LDGLayerWeight *layer_weights, const void *final_norm_weight,
    const void *lm_head_weight, const void *cos_table, const void *sin_table,
    void *k_cache, void *v_cache, void *hidden_buffer, void *g_normalized,
    void *block_max_vals, void *block_max_idxs, int *output_log, int num_layers,
    int start_position, int max_seq_len, float attn_scale, int eos_token_id,
    int synchronize, cudaStream_t stream);
int qmk_prefill(
    const int *token_ids_host, int num_tokens, const void *embed_weight,
    const struct LDGLayerWeight *layer_weights, const void *final_norm_weight,
    const void *cos_table, const void *sin_table, void *k_cache, void *v_cache,
    int num_layers, int start_position, int max_seq_len, float attn_scale,
    cudaStream_t stream);

/* Greedy decode of up to four independent sequences in ONE persistent launch:
 * every weight row is streamed from HBM once per step and used by all
 * sequences; the math warps of each CTA are split into one group per sequence.
 * The reference decodes one sequence per launch (megakernel_5090.cu:1216-1260
 * launch_ldg_generate_nosync); this is its multi-sequence form, the building
 * block for the batched configurations.  Host arrays of num_sequences entries:
 * first_token_ids, start_positions (each sequence's own cache length), and the
 * DEVICE pointers k_caches / v_caches (one cache pair per sequence, same
 * [layer][8][max_seq_len][128] fp16 shape, filled by qmk_prefill) and
 * output_logs (num_steps ints each).  All sequences run num_steps steps; there
 * is no EOS stop (cut the logs on the host).  With a logits dump set
 * (qmk_set_logits_dump) the buffer is [sequence][step][vocab].  num_sequences
 * is 1, 2, 3 or 4; two sequences may not share a cache or a log. */
int qmk_generate_batch(
    int num_sequences, const int *first_token_ids, const int *start_positions,
    int num_steps, const void *embed_weight,
    const struct LDGLayerWeight *layer_weights, const void *final_norm_weight,
    const void *lm_head_weight, const void *cos_table, const void *sin_table,
    void *const *k_caches, void *const *v_caches, int *const *output_logs,
    int num_layers, int max_seq_len, float attn_scale, int synchronize,
    cudaStream_t stream);

/* qmk_generate for callers that cannot allocate device memory while running -
 * for example a server that handed all free HBM to its own cache pool when it
 * started, or a loop that must not hit cudaMalloc's device-wide
 * synchronisation.  It has no counterpart in the reference.  It runs the same
 * kernel and gives the same tokens, but its scratch (exchange words, fp32
 * rotary table, status) is a fixed 1,542,208-byte device array inside the
 * library, held on every GPU the process uses until exit; the call and
 * everything under it make no cudaMalloc / cudaFree / cudaHostAlloc.
 * Limits: max_seq_len <= 2048 (the rotary table's size; a larger value is
 * refused with QMK_ERR_BAD_ARGUMENT and a message), num_layers <= 48.
 * The first call on a device looks up the array's device address and sets the
 * kernel's shared-memory attribute: make that call before any stream capture.
 * Every call blocks until the stream is idle (it reads the kernel's status word
 * back into host memory).  The array is part of the library's CUDA module, which
 * the runtime loads on first use: a process that is about to hand all free HBM
 * to its own pool should touch the library first (qmk_num_ctas() is enough).
 * All calls on a device share the array, which keeps the previous call's
 * contents (status and rotary table are rewritten per call, exchange words
 * are distinguished by tags): calls that overlap on the GPU race.  Blocks
 * until the stream is idle; vocab/split/time-out options come from
 * qmk_configure; RoPE always uses in-kernel fp32 angles. */
int qmk_generate_static(
    int first_token_id, int num_steps, const void *embed_weight,
    const struct LDGLayerWeight *layer_weights, const void *final_norm_weight,
    const void *lm_head_weight, void *k_cache, void *v_cache, void *g_normalized,
    int *output_log, int num_layers, int start_position, int max_seq_len,
    float attn_scale, int eos_token_id, cudaStream_t stream);

/* qmk_prefill on the tensor cores: the prompt is processed in chunks of up to 4096 tokens; per layer the
 * seven projections run as tcgen05 GEMMs over the whole chunk (weights are read once per chunk instead
 * of once per token, megakernel_5090.cu:1324-1350), with row-wise kernels for RMSNorm, per-head QK-norm +
 * RoPE + cache write, causal attention over the cache, and SwiGLU between them.  Same arguments, cache
 * layout, position rule and blocking behaviour as qmk_prefill; all three weight formats (packed FP8 / NVFP4 matrices
 * stay packed in HBM and are expanded to fp16 tiles inside the GEMM, see qmk_gemm_packed_tn).  GEMM operands are rounded to fp16 (the
 * decode kernel keeps fp32 activations), so cache rows agree with qmk_prefill's to fp16 rounding, not
 * bit for bit.  Scratch (about 230 MB) is allocated on the first call per device. */
int qmk_prefill_chunked(
    const int *token_ids_host, int num_tokens, const void *embed_weight,
    const struct LDGLayerWeight *layer_weights, const void *cos_table, const void *sin_table,
    void *k_cache, void *v_cache, int num_layers, int start_position, int max_seq_len,
    float attn_scale, cudaStream_t stream);

/* Several prompts in ONE pass of qmk_prefill_chunked (no counterpart in the reference, whose prefill is one sequence;
 * the continuous-batching caller admits waiting requests together): sequence s has seq_lens[s] tokens - all of them
 * concatenated in token_ids_host - and its own caches k_caches[s] / v_caches[s] (HOST arrays of device pointers, the
 * layout of qmk_prefill), filled from position 0.  The sequences become consecutive row ranges of one chunk, each
 * padded to whole 128-row tiles (at most 64 sequences and 4096 padded rows per call); the GEMMs and row kernels run
 * once over all rows, the attention kernel takes (sequence, query tile, head) items and reads each sequence's cache
 * through its own tensor map.  Needs the tcgen05 attention kernel (qmk_set_prefill_attention(1), the default).  Every
 * cache ends up as qmk_prefill_chunked would have left it, to the rounding of a different GEMM tiling.  Blocks. */
int qmk_prefill_packed(
    const int *token_ids_host, int num_seqs, const int *seq_lens, const void *embed_weight,
    const struct LDGLayerWeight *layer_weights, const void *cos_table, const void *sin_table,
    void *const *k_caches, void *const *v_caches, int num_layers, int max_seq_len,
    float attn_scale, cudaStream_t stream);

/* Greedy decode of up to 128 sequences on the tensor-core path (the batched configurations): each step runs
 * the seven projections and the LM head as tcgen05 GEMMs over one 128-row tile of sequences, with row kernels
 * for the norms, per-head QK-norm + RoPE + cache write (each sequence at its own position in its own cache),
 * per-sequence attention over the cache, SwiGLU and the argmax.  Same arguments as qmk_generate_batch (host
 * arrays of num_sequences entries; no EOS stop; logits dump [sequence][step][vocab]); all three weight formats
 * (packed matrices are expanded inside the GEMMs, which halves / quarters the weight bytes of a step), vocab
 * a multiple of 128; blocks until done.  One step costs about 400 kernel launches, so it pays from roughly
 * eight sequences on; below that qmk_generate_batch (one persistent launch) is faster.  Numerics as
 * qmk_prefill_chunked (GEMM operands rounded to fp16). */
int qmk_decode_batched(
    int num_sequences, const int *first_token_ids, const int *start_positions,
    int num_steps, const void *embed_weight,
    const struct LDGLayerWeight *layer_weights, const void *final_norm_weight,
    const void *lm_head_weight, const void *cos_table, const void *sin_table,
    void *const *k_caches, void *const *v_caches, int *const *output_logs,
    int num_layers, int max_seq_len, float attn_scale, cudaStream_t stream);

/* C[m x n] (fp32, row-major, DEVICE) = A[m x k] * B[n x k]^T with fp16 row-major DEVICE operands, on the
 * tcgen05 tensor cores (TMA-fed, accumulator in TMEM).  m and n multiples of 128, k a multiple of 64,
 * operands 16-byte aligned.  This is the GEMM the chunked prefill is built from; the reference has no
 * counterpart (its prefill repeats the decode kernels once per prompt token, megakernel_5090.cu:1324-1350).
 * Blocks until done. */
int qmk_gemm_f16_tn(const void *a, const void *b, float *c, int m, int n, int k, cudaStream_t stream);

/* The same GEMM with B kept PACKED in device memory: weight_format 1 = FP8-E4M3 rows (k bytes + 16-byte trailer with
 * the fp32 row scale), 2 = NVFP4 rows (k/2 bytes of e2m1 pairs, low nibble first; k/16 e4m3 block-16 scales; 16-byte
 * trailer with the fp32 tensor scale).  The packed K blocks cross HBM as they are and are expanded to fp16 tiles in
 * shared memory inside the kernel (e4m3 and e2m1 x block scale are exact in fp16), the fp32 scale multiplies the
 * accumulator: products are those of the dequantised matrix with fp16 activations, fp32 accumulation.  k <= 3072,
 * a multiple of 64 (NVFP4: of 256, so that rows stay 16-byte aligned).
 * mode 0: c fp32 [m x n].  mode 1: split-K by four, c fp32 [4][m x n] partial matrices.  mode 2: b = gate, b2 = up,
 * c fp16 [m x n] = silu(a gate^T) * (a up^T).  box_n: rows of B per CTA (32, 64, 128; modes 1 and 2: 32 or 64), 0 picks.
 * These are the three forms qmk_decode_batched and qmk_prefill_chunked use when a packed weight format is selected.
 * No counterpart in the reference (fp16 only).  Blocks until done. */
int qmk_gemm_packed_tn(const void *a, const void *b, const void *b2, void *c, int m, int n, int k, int weight_format,
                       int mode, int box_n, cudaStream_t stream);

/* Synchronises the device and returns the status word of the last launch
 * (QMK_OK, or the first error a CTA recorded). */
int qmk_sync_status(void);
/* Text of the last error on this thread's device ("" if none). */
const char *qmk_last_error(void);
/* Persistent grid size (CTAs) and bytes of library-owned device scratch. */
int qmk_num_ctas(void);
long long qmk_scratch_bytes(void);
/* Runs one bounded wait on a word nothing ever sets, with budget_us
 * microseconds; returns QMK_ERR_WAIT_TIMEOUT when the wait gave up as designed. */
int qmk_selftest_wait_timeout(int budget_us);

/* The same for the tcgen05 GEMM: one tile whose loads are never issued; the MMA thread's wait runs out after
 * budget_us, all roles leave, TMEM is freed; returns QMK_ERR_WAIT_TIMEOUT when that happened as designed. */
int qmk_selftest_gemm_wait_timeout(int budget_us);

#ifdef __cplusplus
}
#endif
#endif /* QWEN_MEGAKERNEL_H_ */
