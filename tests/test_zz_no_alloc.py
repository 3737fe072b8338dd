"""GPU test of the allocation-free entry point ``qmk_generate_static`` (collected last on purpose).

Some users of this library cannot allocate device memory at the moment they want to decode: a serving
process that handed every free byte of HBM to its own cache pool when it started, or a latency-critical
loop that cannot take the device-wide synchronisation a cudaMalloc implies.  For them the library has one
entry point whose scratch is a fixed device array inside the library.  This test drives it through the C ABI
and checks that it produces what the ordinary entry point produces - same greedy tokens, logits and
final-norm vector within the tolerance the other parity tests use - on two calls in a row (the second call
meets the array as the first one left it), and that a context beyond the array's limit is refused.
"""

import pytest
import torch

import synthetic as S

pytestmark = pytest.mark.gpu
LOGIT_TOL = 3e-2   # same bound as tests/test_gpu_parity.py


def test_static_scratch_entry_point_matches_allocating_one(built_library):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import qwen_megakernel_C as C
    from Model.Qwen06B_architecture import Decoder

    vocab, layers, max_seq, steps = 4096, 2, 64, 6
    w = S.make_weights(seed=3, num_layers=layers, vocab_size=vocab, norm_std=0.1, max_seq_len=max_seq)
    ids = S.make_prompt(12, seed=5, vocab_size=vocab)
    eng = Decoder(weights=S.weights_to(w, "cuda"), verbose=False, max_seq_len=max_seq)

    # the ordinary (allocating) entry point: prefill, then `steps` greedy tokens with all logits dumped
    ref_logits = torch.zeros(steps, vocab, device="cuda")
    C.set_logits_dump(ref_logits)
    try:
        ref_tokens = eng.generate_ids(ids, steps)
    finally:
        C.set_logits_dump(None)
    ref_normed = eng._norm_out.clone()
    start = len(ids) - 1                      # cache rows 0..start-1 hold the prompt; decode rewrites the rest
    assert len(ref_tokens) == steps

    for call in range(2):                     # twice in a row: the second call reuses the array as left behind
        log = torch.full((steps,), -1, dtype=torch.int32, device="cuda")
        normed = torch.zeros(1024, device="cuda")
        logits = torch.zeros(steps, vocab, device="cuda")
        C.set_logits_dump(logits)
        try:
            C.generate_static(ids[-1], steps, eng._embed_weight, eng._layer_weights_packed, eng._final_norm_weight,
                              eng._lm_head_weight, eng._k_cache, eng._v_cache, normed, log, layers, start, max_seq,
                              eng._attn_scale, -1)
        finally:
            C.set_logits_dump(None)
        assert log.cpu().tolist() == ref_tokens, f"call {call}"
        assert float((logits - ref_logits).abs().max()) < LOGIT_TOL, f"call {call}"
        assert float((normed - ref_normed).abs().max()) < LOGIT_TOL, f"call {call}"

    # sizes beyond the fixed array are refused with a clear message, and nothing is launched
    with pytest.raises(RuntimeError, match="static scratch limit"):
        C.generate_static(ids[-1], 1, eng._embed_weight, eng._layer_weights_packed, eng._final_norm_weight,
                          eng._lm_head_weight, eng._k_cache, eng._v_cache, None,
                          torch.zeros(1, dtype=torch.int32, device="cuda"), layers, 0, 4096, eng._attn_scale, -1)
    # the ordinary path is unaffected
    assert eng.generate_ids(ids, steps) == ref_tokens
