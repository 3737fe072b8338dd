// Launch parameters and the per-layer pointer record shared by the builds of the decode megakernel.
#ifndef QMK_MEGAKERNEL_PARAMS_H_
#define QMK_MEGAKERNEL_PARAMS_H_

#include <cuda_fp16.h>
#include <stdint.h>

namespace qmkp {

// Same binary layout as the reference's per-layer pointer record
// (megakernel_5090.cu:91-104): 11 fp16 pointers + 1 pad = 96 bytes.
struct __align__(16) LayerW {
  const __half *in_ln, *wq, *wk, *wv, *q_norm, *k_norm, *wo, *post_ln, *w_gate, *w_up, *w_down;
  const void *pad;
};

// K-major copies of the two projections whose input is produced slice by slice (O: the attention output, down:
// the MLP activations).  The library makes them from the caller's [out,in] matrices: row e of wo_t holds
// W_o[:, e], row m of wd_t holds W_down[:, m] (1024 outputs each), so that the rows a CTA needs for ITS slice of
// the input form one contiguous range.  fp8 format: 1024 e4m3 bytes per row, the per-output fp32 scales of the
// matrix follow the last row.
struct __align__(16) LayerT {
  const void *wo_t, *wd_t;
};

constexpr int MAX_SEQ = 4;       // sequences one launch of the multi-sequence build can carry

struct Params {
  const __half *embed;
  const LayerW *layers;
  const __half *final_norm;
  const __half *lm_head;
  const __half *cos_table, *sin_table;
  const float *rope;             // fp32 [position][cos 64 | sin 64], built by rope_table_kernel
  __half *k_cache, *v_cache;
  unsigned long long *ll;
  unsigned int *status;          // [0] code, [1] where, [2] cta
  const int *token_ids;          // prefill: device array of num_steps tokens
  int *output_log;               // decode: token per step (may be null)
  int *output_token;             // decode: last token (may be null)
  float *normalized_out;         // fp32[1024] final-norm output of the last step (may be null)
  __half *hidden_out;            // fp16[1024] last hidden state (may be null)
  float *bmax_vals;              // per-CTA argmax partials (may be null)
  int *bmax_idxs;
  float *logits_out;             // debug dump (may be null)
  unsigned long long *prof;      // debug: per-CTA phase timestamps of the last step (may be null)
  unsigned long long timeout_ns;
  int first_token, num_steps, num_layers, start_position, max_seq_len, vocab;
  int eos, prefill, rope_from_table, split_len;
  unsigned int seq_base;
  float attn_scale;
  int spin_sleep_ns;             // back-off between polls of an exchange word (0 = none)
  int l2_evict_first;            // weight stream L2 policy: 1 evict_first, 0 default
  int wfmt;                      // weight format of all matrices: 0 fp16 rows, 1 fp8-e4m3 rows + 16-byte scale trailer
  int repl;                      // copies of the exchange area (1, 2 or 4); CTA i polls copy i % repl
  int stream_inflight;           // max weight chunks in flight during layer phases (0 = ring depth)
  // Sequences interleaved in one launch (multi-sequence build only; the single-sequence kernel reads
  // the scalar fields above and the host mirrors them into entry 0 for the shared producer code).
  int nseq;                      // 1 .. MAX_SEQ
  int first_tokens[MAX_SEQ];
  int start_positions[MAX_SEQ];
  __half *k_caches[MAX_SEQ], *v_caches[MAX_SEQ];
  int *output_logs[MAX_SEQ];     // decode: token per step of each sequence
  // Fused single-sequence kernel only (null / 0 elsewhere).
  const LayerT *layers_t;        // K-major copies, one record per layer
  unsigned long long *red;       // all-reduce words of the two residual sums, zeroed by the host before the launch
  int red_copies;                // accumulator copies per sum (1 or 2): CTA i adds into copy i % red_copies
  // Tensor-core build: tiled-copy descriptors (CUtensorMap, 128 bytes each) of the K and V caches seen as
  // [layers * 8 * max_seq_len rows][128] fp16, boxes of 16 rows x 64 columns with the 128-byte swizzle.
  alignas(64) unsigned char kmap[128];
  alignas(64) unsigned char vmap[128];
};

}  // namespace qmkp
#endif  // QMK_MEGAKERNEL_PARAMS_H_
