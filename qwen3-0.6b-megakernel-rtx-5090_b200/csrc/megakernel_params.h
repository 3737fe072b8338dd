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
};

}  // namespace qmkp
#endif  // QMK_MEGAKERNEL_PARAMS_H_
