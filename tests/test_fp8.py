"""FP8-E4M3 weight variant: quantiser (CPU) and engine parity against the oracle run on the dequantised
weights (GPU).  Tolerance: identical greedy tokens; logits within max-abs 3e-2 of the oracle on the SAME
quantised weights (the engine and the oracle then differ only in summation order); the distance to the
fp16 model is printed, not asserted - it is a property of the quantisation, not of the engine."""

import pytest
import torch

import quantize as Q
import synthetic as S
from oracle.decoder_ref import Decoder as OracleDecoder


def test_quantiser_scheme_and_row_format():
    g = torch.Generator("cpu").manual_seed(0)
    w = (torch.randn(6, 64, generator=g) * 0.02).to(torch.float16)
    w[3] = 0                                                  # an all-zero row must not divide by zero
    q, s = Q.quantize_rows_fp8(w)
    assert q.dtype == torch.float8_e4m3fn and s.dtype == torch.float32 and s.shape == (6,)
    assert torch.allclose(s[:3], w[:3].float().abs().amax(1) / 448.0) and s[3] == 1.0
    deq = Q.dequantize_rows_fp8(q, s)
    # e4m3 has 3 mantissa bits: relative error <= 2^-4 for normal values, absolute error bounded by the scale
    assert ((deq - w.float()).abs() <= w.float().abs() * 2 ** -4 + s[:, None] * 2 ** -9 + 1e-12).all()
    assert deq[3].abs().max() == 0
    assert (deq.abs().amax(1)[:3] - w[:3].float().abs().amax(1)).abs().max() < 1e-6   # the row maximum is exact
    packed = Q.pack_rows_fp8(q, s)
    assert packed.shape == (6, 64 + 16) and packed.dtype == torch.uint8
    assert torch.equal(packed[:, :64], q.view(torch.uint8))
    assert torch.equal(packed[:, 64:68].contiguous().view(torch.float32).flatten(), s)
    assert packed[:, 68:].abs().max() == 0


def test_quantised_weight_dicts_and_byte_count():
    w = S.make_weights(seed=2, num_layers=1, vocab_size=128)
    eng, ora = Q.quantize_weights_fp8(w)
    assert eng["lm_head_weight"] is eng["embed_weight"] and ora["lm_head_weight"] is ora["embed_weight"]
    assert eng["embed_weight"].shape == (128, 1024 + 16)
    shapes = [tuple(t.shape) for t in eng["layer_weights"]]
    assert shapes[1] == (2048, 1040) and shapes[6] == (1024, 2064) and shapes[10] == (1024, 3088)
    assert eng["layer_weights"][0].dtype == torch.float16          # norm vectors untouched
    assert ora["layer_weights"][1].dtype == torch.float32
    # ~598 MB per decode step for the full model (598.1 M with bare fp32 row scales and no 16-byte trailers)
    assert 0.595e9 < Q.weight_bytes_fp8() < 0.610e9


@pytest.mark.gpu
def test_fp8_engine_matches_oracle_on_dequantised_weights(built_library):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import qwen_megakernel_C as C
    from Model.Qwen06B_architecture import Decoder
    vocab, steps = 4096, 8
    w = S.make_weights(seed=3, num_layers=2, vocab_size=vocab, norm_std=0.1, max_seq_len=64)
    ids = S.make_prompt(12, seed=5, vocab_size=vocab)
    eng_w, ora_w = Q.quantize_weights_fp8(w)
    want, logits = OracleDecoder(ora_w, max_seq_len=64).generate_ids(ids, steps, keep_logits=True)
    _, logits16 = OracleDecoder(w, max_seq_len=64).generate_ids(ids, steps, keep_logits=True)
    eng = Decoder(weights=S.weights_to(eng_w, "cuda"), verbose=False, max_seq_len=64, weight_format="fp8")
    dump = torch.zeros(steps, vocab, device="cuda")
    C.set_logits_dump(dump)
    try:
        got = eng.generate_ids(ids, steps)
        again = eng.generate_ids(ids, steps)
    finally:
        C.set_logits_dump(None)
        C.set_weight_format("fp16")
    err = float((dump.cpu() - logits).abs().max())
    dq = float((logits - logits16).abs().max())
    print(f"fp8: max |logit - oracle(fp8 weights)| = {err:.3e}; quantisation moved the logits by up to {dq:.3e}")
    assert got == want and again == want
    assert err < 3e-2


@pytest.mark.gpu
def test_fp8_full_model_greedy_tokens(built_library):
    """Full Qwen3-0.6B shape, fp8 weights, 32-token prompt, 16 greedy steps against the oracle on the
    dequantised weights."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import qwen_megakernel_C as C
    from Model.Qwen06B_architecture import Decoder
    w = S.make_weights(seed=0, max_seq_len=128)
    ids = S.make_prompt(32, seed=0)
    eng_w, ora_w = Q.quantize_weights_fp8(w)
    want, logits = OracleDecoder(ora_w, max_seq_len=128).generate_ids(ids, 16, keep_logits=True)
    margins = torch.topk(logits, 2, dim=-1).values
    min_margin = float((margins[:, 0] - margins[:, 1]).min())
    eng = Decoder(weights=S.weights_to(eng_w, "cuda"), verbose=False, max_seq_len=128, weight_format="fp8")
    dump = torch.zeros(16, S.VOCAB_SIZE, device="cuda")
    C.set_logits_dump(dump)
    try:
        got = eng.generate_ids(ids, 16)
    finally:
        C.set_logits_dump(None)
        C.set_weight_format("fp16")
    err = float((dump.cpu() - logits).abs().max())
    print(f"fp8 full: max |logit - oracle| = {err:.3e}; min greedy margin {min_margin:.3e}")
    assert err < 3e-2
    assert got == want


@pytest.mark.gpu
def test_fp8_four_sequences_per_launch(built_library):
    """FP8 weights through the multi-sequence launch (the B = 4 shape of the FP8 configuration): every
    sequence against the oracle on the dequantised weights."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import qwen_megakernel_C as C
    from Model.Qwen06B_architecture import BatchDecoder
    vocab, steps = 4096, 6
    w = S.make_weights(seed=3, num_layers=2, vocab_size=vocab, norm_std=0.1, max_seq_len=16)
    eng_w, ora_w = Q.quantize_weights_fp8(w)
    lens = [40, 300, 9, 150]
    prompts = [S.make_prompt(L, seed=70 + i, vocab_size=vocab) for i, L in enumerate(lens)]
    eng = BatchDecoder(weights=S.weights_to(eng_w, "cuda"), tokenizer=S.StubTokenizer(-1, vocab), num_sequences=4,
                       max_seq_len=384, weight_format="fp8")
    dump = torch.zeros(4, steps, vocab, device="cuda")
    C.set_logits_dump(dump)
    try:
        got = eng.generate_ids(prompts, steps)
    finally:
        C.set_logits_dump(None)
        C.set_weight_format("fp16")
    for b in range(4):
        want, logits = OracleDecoder(ora_w, max_seq_len=384).generate_ids(prompts[b], steps, keep_logits=True)
        err = float((dump[b].cpu() - logits).abs().max())
        print(f"fp8 batch 4, sequence {b}: max |logit - oracle(fp8 weights)| = {err:.3e}")
        assert got[b] == want
        assert err < 3e-2


def test_nvfp4_quantiser_scheme():
    g = torch.Generator("cpu").manual_seed(1)
    w = (torch.randn(5, 64, generator=g) * 0.02).to(torch.float16)
    w[2] = 0
    vals, sb, st = Q.quantize_blocks_nvfp4(w)
    assert sb.dtype == torch.float8_e4m3fn and sb.shape == (5, 4) and st > 0
    assert set(vals.abs().unique().tolist()) <= set(Q.E2M1_GRID)
    deq = Q.dequantize_nvfp4(vals, sb, st)
    assert deq[2].abs().max() == 0
    # e2m1 spacing is at most 2 on a scale of 6: error <= 1/6 of the block maximum (+ the e4m3 scale rounding)
    blocks = w.float().view(5, 4, 16)
    bound = blocks.abs().amax(dim=2, keepdim=True) * (1 / 6 + 1 / 8)
    assert ((deq.view(5, 4, 16) - blocks).abs() <= bound + 1e-9).all()
    # ties go to the even code: 0.25 -> 0, 0.75 -> 1, 2.5 -> 2, 5 -> 4
    assert Q.round_to_e2m1(torch.tensor([0.25, 0.75, 2.5, 5.0, -1.25, 7.0])).tolist() == [0.0, 1.0, 2.0, 4.0, -1.0, 6.0]
    assert 0.33e9 < Q.weight_bytes_nvfp4() < 0.34e9


@pytest.mark.gpu
@pytest.mark.parametrize("fmt,n", [("fp8", 16), ("nvfp4", 64)])
def test_quantised_models_on_the_batched_tensor_core_path(built_library, fmt, n):
    """The B = 16 FP8 and B = 64 NVFP4 configurations' shapes with the weights PACKED in device memory (expanded to
    fp16 tiles inside the GEMMs) and the tensor-core prefill on the same packed matrices: every sequence against
    the oracle on the dequantised weights (logits within 3e-2; tokens equal wherever the oracle's greedy margin
    exceeds twice the logit error)."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import qwen_megakernel_C as C
    from Model.Qwen06B_architecture import BatchDecoder
    vocab, steps, L = 2048, 4, 192
    w = S.make_weights(seed=31, num_layers=2, vocab_size=vocab, norm_std=0.1, max_seq_len=16)
    eng_w, ora_w = (Q.quantize_weights_fp8 if fmt == "fp8" else Q.quantize_weights_nvfp4)(w)
    lens = [1 + (17 * i) % 150 for i in range(n)]
    prompts = [S.make_prompt(Ln, seed=600 + i, vocab_size=vocab) for i, Ln in enumerate(lens)]
    eng = BatchDecoder(weights=S.weights_to(eng_w, "cuda"), tokenizer=S.StubTokenizer(-1, vocab), num_sequences=n,
                       max_seq_len=L, engine="gemm", prefill_mode="tensor", weight_format=fmt)
    dump = torch.zeros(n, steps, vocab, device="cuda")
    C.set_logits_dump(dump)
    try:
        got = eng.generate_ids(prompts, steps)
    finally:
        C.set_logits_dump(None)
        C.set_weight_format("fp16")
    dump = dump.cpu()
    worst, equal = 0.0, 0
    for b in range(n):
        want, logits = OracleDecoder(ora_w, max_seq_len=L).generate_ids(prompts[b], steps, keep_logits=True)
        for s in range(steps):
            err = float((dump[b, s] - logits[s]).abs().max())
            worst = max(worst, err)
            assert err < 3e-2
            if got[b][s] != want[s]:
                top2 = logits[s].topk(2).values
                assert float(top2[0] - top2[1]) < 2 * err + 1e-6
                break
            equal += 1
    print(f"{fmt} packed, {n} sequences: worst max |logit - oracle| = {worst:.3e}; {equal}/{n * steps} steps token-equal")
    assert equal >= 0.9 * n * steps    # near-ties (margin below twice the logit error) may break a sequence off early
