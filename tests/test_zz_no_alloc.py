"""GPU test of the allocation-free entry point ``qmk_generate_static`` (collected last on purpose).

Some users of this library cannot allocate device memory at the moment they want to decode: a serving
process that handed every free byte of HBM to its own cache pool when it started, or a latency-critical
loop that cannot take the device-wide synchronisation a cudaMalloc implies.  For them the library has one
entry point whose scratch is a fixed device array inside the library.  This test drives it through the C ABI
and checks that it produces what the ordinary entry point produces - same greedy tokens, logits and
final-norm vector within the tolerance the other parity tests use - on two calls in a row (the second call
meets the array as the first one left it), and that a context beyond the array's limit is refused.
"""

import json
import os
import subprocess
import sys

import numpy as np
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
    # ... and the CPU oracle's golden file for this model (same seeds): the entry point is checked against the
    # oracle itself, not only against its sibling
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "tiny_l2_v4096.npz"))
    assert g["prompt"].tolist() == ids and g["tokens"].tolist()[:steps] == ref_tokens
    gold_logits = torch.from_numpy(g["logits"][:steps]).cuda()

    for call in range(2):                     # twice in a row: the second call reuses the array as left behind
        log = torch.full((steps,), -1, dtype=torch.int32, device="cuda")
        normed = torch.zeros(1024, device="cuda")
        logits = torch.zeros(steps, vocab, device="cuda")
        C.set_logits_dump(logits)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        try:
            C.generate_static(ids[-1], steps, eng._embed_weight, eng._layer_weights_packed, eng._final_norm_weight,
                              eng._lm_head_weight, eng._k_cache, eng._v_cache, normed, log, layers, start, max_seq,
                              eng._attn_scale, -1)
        finally:
            C.set_logits_dump(None)
        if call == 1:   # the first call may load the library's module (its array included); later calls take nothing
            assert torch.cuda.mem_get_info()[0] == free_before, "the allocation-free entry point took device memory"
        assert log.cpu().tolist() == ref_tokens, f"call {call}"
        assert float((logits - ref_logits).abs().max()) < LOGIT_TOL, f"call {call}"
        assert float((logits - gold_logits).abs().max()) < LOGIT_TOL, f"call {call}: against the oracle"
        assert float((normed - ref_normed).abs().max()) < LOGIT_TOL, f"call {call}"

    # sizes beyond the fixed array are refused with a clear message, and nothing is launched
    with pytest.raises(RuntimeError, match="static scratch limit"):
        C.generate_static(ids[-1], 1, eng._embed_weight, eng._layer_weights_packed, eng._final_norm_weight,
                          eng._lm_head_weight, eng._k_cache, eng._v_cache, None,
                          torch.zeros(1, dtype=torch.int32, device="cuda"), layers, 0, 4096, eng._attn_scale, -1)
    # the ordinary path is unaffected
    assert eng.generate_ids(ids, steps) == ref_tokens


def test_static_scratch_entry_point_with_fp8_rows(built_library):
    """The same entry point on FP8-E4M3 rows (per-row scale in the row trailer): tokens equal to the oracle run on the
    dequantised weights, twice in a row."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import quantize
    import qwen_megakernel_C as C
    from Model.Qwen06B_architecture import Decoder
    from oracle.decoder_ref import Decoder as Oracle

    vocab, layers, max_seq, steps = 4096, 2, 64, 6
    w = S.make_weights(seed=3, num_layers=layers, vocab_size=vocab, norm_std=0.1, max_seq_len=max_seq)
    ids = S.make_prompt(12, seed=5, vocab_size=vocab)
    eng_w, oracle_w = quantize.quantize_weights_fp8(w)
    want = Oracle(oracle_w, max_seq_len=max_seq).generate_ids(ids, steps)[0]
    try:
        eng = Decoder(weights=S.weights_to(eng_w, "cuda"), verbose=False, max_seq_len=max_seq, weight_format="fp8")
        assert eng.generate_ids(ids, steps) == want          # fills cache rows 0..len(ids)-2 too
        for call in range(2):
            log = torch.full((steps,), -1, dtype=torch.int32, device="cuda")
            C.generate_static(ids[-1], steps, eng._embed_weight, eng._layer_weights_packed, eng._final_norm_weight,
                              eng._lm_head_weight, eng._k_cache, eng._v_cache, None, log, layers, len(ids) - 1, max_seq,
                              eng._attn_scale, -1)
            assert log.cpu().tolist() == want, f"call {call}"
    finally:
        C.set_weight_format("fp16")


COLD_START = r"""
import json, sys
sys.path[:0] = [{root!r}, {pkg!r}]
import numpy as np, torch
import synthetic as S
import qwen_megakernel_C as C                      # nothing else of the package: no Decoder, no allocating call before
from Model.Qwen06B_architecture import _pack_layer_weights
g = np.load({golden!r})
vocab, layers, max_seq, steps = 4096, 2, 64, 6
w = S.weights_to(S.make_weights(seed=3, num_layers=layers, vocab_size=vocab, norm_std=0.1, max_seq_len=max_seq), "cuda")
table = _pack_layer_weights(w["layer_weights"])
k = torch.zeros(layers, 8, max_seq, 128, dtype=torch.float16, device="cuda"); v = torch.zeros_like(k)
C.configure(vocab_size=vocab)
ids = g["prompt"].tolist()
one = torch.zeros(1, dtype=torch.int32, device="cuda")
for pos, t in enumerate(ids[:-1]):                  # the prompt, one decode step per token: fills the cache
    C.generate_static(t, 1, w["embed_weight"], table, w["final_norm_weight"], w["lm_head_weight"], k, v, None, one, layers, pos, max_seq, 128 ** -0.5, -1)
log = torch.full((steps,), -1, dtype=torch.int32, device="cuda")
C.generate_static(ids[-1], steps, w["embed_weight"], table, w["final_norm_weight"], w["lm_head_weight"], k, v, None, log, layers, len(ids) - 1, max_seq, 128 ** -0.5, -1)
print(json.dumps(dict(tokens=log.cpu().tolist(), want=g["tokens"].tolist()[:steps])))
"""


def test_static_scratch_entry_point_as_first_call_of_a_process(built_library):
    """The advertised use: a process whose FIRST call into the library is the allocation-free entry point (so its
    own set-up branch runs: symbol lookup, kernel attributes, default RoPE frequencies), with caller-allocated
    tensors only.  Tokens are compared with the CPU oracle's golden file."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    pkg = os.path.join(root, "qwen3-0.6b-megakernel-rtx-5090_b200")
    golden = os.path.join(root, "tests", "golden", "tiny_l2_v4096.npz")
    proc = subprocess.run([sys.executable, "-c", COLD_START.format(root=root, pkg=pkg, golden=golden)],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-4000:]
    res = json.loads(proc.stdout.strip().splitlines()[-1])
    assert res["tokens"] == res["want"]
