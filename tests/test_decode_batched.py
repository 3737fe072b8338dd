"""Batched decode on the tensor-core path (``decode_batched`` / ``BatchDecoder(engine="gemm")``) against the CPU
oracle, sequence by sequence.  GEMM operands are rounded to fp16 on this path (the oracle and the persistent
kernel keep fp32 activations), so the bar is the stated tolerance: logits within 3e-2 max-abs of the oracle's,
and - on these seeds - identical greedy tokens."""

import json
import os

import pytest
import torch

import synthetic as S
from oracle.decoder_ref import Decoder as OracleDecoder

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
LOGIT_TOL = 3e-2


@pytest.fixture(scope="module")
def C(built_library):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import qwen_megakernel_C
    return qwen_megakernel_C


def _engine(w, n, max_seq_len, **kw):
    from Model.Qwen06B_architecture import BatchDecoder
    return BatchDecoder(weights=S.weights_to(w, "cuda"), tokenizer=S.StubTokenizer(-1, w["embed_weight"].shape[0]),
                        num_sequences=n, max_seq_len=max_seq_len, **kw)


@pytest.mark.parametrize("n", [1, 5, 19, 40])
def test_tiny_model_against_oracle(C, n):
    """Sequence counts that are no multiple of anything; contexts from 1 token to several rounds of the attention
    kernels, all different.  40 sequences take the bulk-copy-fed attention kernel (its 6-slot ring wraps from 193
    cache rows on)."""
    vocab, steps, L = 2048, 5, 768
    w = S.make_weights(seed=21, num_layers=3, vocab_size=vocab, norm_std=0.1, max_seq_len=16)
    lens = [(1 + 37 * i * i) % 700 + 1 for i in range(n)]
    prompts = [S.make_prompt(Ln, seed=300 + i, vocab_size=vocab) for i, Ln in enumerate(lens)]
    eng = _engine(w, n, L, engine="gemm")
    dump = torch.zeros(n, steps, vocab, device="cuda")
    C.set_logits_dump(dump)
    try:
        got = eng.generate_ids(prompts, steps)
    finally:
        C.set_logits_dump(None)
    worst = 0.0
    for b in range(n):
        want, logits = OracleDecoder(w, max_seq_len=L).generate_ids(prompts[b], steps, keep_logits=True)
        err = float((dump[b].cpu() - logits).abs().max())
        worst = max(worst, err)
        assert got[b] == want, f"sequence {b} (prompt {lens[b]} tokens)"
        assert err < LOGIT_TOL
    print(f"decode_batched, {n} sequences: worst max |logit - oracle| = {worst:.3e}")
    assert eng.positions[:n] == [Ln - 1 + steps for Ln in lens]


def test_long_contexts_split_over_several_ctas(C):
    """Two sequences: the attention kernel divides each sequence's cache rows among eight CTAs (nine ring chunks
    per CTA at 2300 tokens, more than the ring has slots) and the last CTA to arrive adds the partial states."""
    vocab, steps, L = 2048, 4, 2432
    w = S.make_weights(seed=23, num_layers=2, vocab_size=vocab, norm_std=0.1, max_seq_len=16)
    lens = [2300, 901]
    prompts = [S.make_prompt(Ln, seed=450 + i, vocab_size=vocab) for i, Ln in enumerate(lens)]
    eng = _engine(w, 2, L, engine="gemm", prefill_mode="serial")
    dump = torch.zeros(2, steps, vocab, device="cuda")
    C.set_logits_dump(dump)
    try:
        got = eng.generate_ids(prompts, steps)
    finally:
        C.set_logits_dump(None)
    for b in range(2):
        want, logits = OracleDecoder(w, max_seq_len=L).generate_ids(prompts[b], steps, keep_logits=True)
        err = float((dump[b].cpu() - logits).abs().max())
        print(f"split attention, {lens[b]}-token context: max |logit - oracle| = {err:.3e}")
        assert got[b] == want and err < LOGIT_TOL
    # a second call reuses the arrival counters the first one left at zero
    assert eng.generate_ids(prompts, steps) == got


def test_both_engines_and_tensor_prefill_agree(C):
    """Four sequences through the persistent launch and through the GEMM path (with tensor-core prefill):
    same tokens."""
    vocab, steps, L = 2048, 6, 512
    w = S.make_weights(seed=22, num_layers=2, vocab_size=vocab, norm_std=0.1, max_seq_len=16)
    prompts = [S.make_prompt(Ln, seed=400 + i, vocab_size=vocab) for i, Ln in enumerate([300, 2, 77, 190])]
    a = _engine(w, 4, L, engine="persistent").generate_ids(prompts, steps)
    b = _engine(w, 4, L, engine="gemm", prefill_mode="tensor").generate_ids(prompts, steps)
    assert a == b


def test_full_model_sixteen_sequences(C, full_cfg):
    """Qwen3-0.6B shape, 16 sequences (the B = 16 configuration's shape).  Sequence 0 is the golden prompt;
    the others are compared with the single-sequence engine where its greedy margin allows a verdict."""
    from Model.Qwen06B_architecture import Decoder
    g = json.load(open(os.path.join(GOLDEN, "full_seed0_prompt32.json")))
    w = S.make_weights(seed=full_cfg["seed"], num_layers=28, vocab_size=S.VOCAB_SIZE, max_seq_len=16)
    prompts = [g["prompt"]] + [S.make_prompt(5 + 11 * i, seed=500 + i) for i in range(15)]
    steps = 12
    eng = _engine(w, 16, 256, engine="gemm")
    dump = torch.zeros(16, steps, S.VOCAB_SIZE, device="cuda")
    C.set_logits_dump(dump)
    try:
        got = eng.generate_ids(prompts, steps)
    finally:
        C.set_logits_dump(None)
    assert got[0] == g["tokens"][:steps]
    single = Decoder(weights=eng._base._weights, tokenizer=S.StubTokenizer(-1), verbose=False, max_seq_len=256)
    ref_dump = torch.zeros(steps, S.VOCAB_SIZE, device="cuda")
    worst, checked = 0.0, 0
    for b in range(16):
        C.set_logits_dump(ref_dump)
        try:
            want = single.generate_ids(prompts[b], steps)
        finally:
            C.set_logits_dump(None)
        # compare step by step while the two runs still see the same history
        for s in range(steps):
            err = float((dump[b, s] - ref_dump[s]).abs().max())
            worst = max(worst, err)
            assert err < LOGIT_TOL
            top2 = ref_dump[s].topk(2).values
            margin = float(top2[0] - top2[1])
            if got[b][s] != want[s]:
                assert margin < 2 * err + 1e-6, f"sequence {b} step {s}: tokens differ with margin {margin:.2e}, err {err:.2e}"
                break
            checked += 1
    print(f"full model, 16 sequences: worst max |logit gemm - logit persistent| = {worst:.3e}; {checked} steps token-equal")
    assert checked >= 16 * steps - 8


def test_step_overlap_changes_nothing_but_time(C):
    """The kernels of a decode step are launched as programmatic dependents of one another (each sets itself up and
    streams its weights behind its predecessor's tail, then waits for it to complete).  Switched off, the same kernels
    run strictly one after the other: tokens and every logit must be bit-identical, through the captured graph and
    through the plain launches of the logits-dump path."""
    vocab, steps, L, n = 2048, 6, 256, 9
    w = S.make_weights(seed=23, num_layers=3, vocab_size=vocab, norm_std=0.1, max_seq_len=16)
    prompts = [S.make_prompt(5 + 23 * i, seed=900 + i, vocab_size=vocab) for i in range(n)]
    eng = _engine(w, n, L, engine="gemm")
    results = {}
    try:
        for overlap in (True, False, True):
            C.set_step_overlap(overlap)
            graph_tokens = eng.generate_ids(prompts, steps)
            dump = torch.zeros(n, steps, vocab, device="cuda")
            C.set_logits_dump(dump)
            try:
                plain_tokens = eng.generate_ids(prompts, steps)
            finally:
                C.set_logits_dump(None)
            assert graph_tokens == plain_tokens
            results.setdefault(overlap, []).append((graph_tokens, dump.cpu()))
    finally:
        C.set_step_overlap(True)
    (tok_on, logit_on), (tok_on2, logit_on2) = results[True]
    (tok_off, logit_off), = results[False]
    assert tok_on == tok_off == tok_on2
    assert torch.equal(logit_on, logit_off) and torch.equal(logit_on, logit_on2)
    want = [OracleDecoder(w, max_seq_len=L).generate_ids(p, steps)[0] for p in prompts]
    assert tok_on == want


@pytest.mark.parametrize("mma", [1, 0])
def test_both_decode_attention_kernels(C, mma):
    """The per-sequence attention of a decode step on mma.sync tiles (default) and on the CUDA-core kernel it replaced:
    contexts of 1 .. 600 rows (chunks of 16 with ragged ends, sequences split over several CTAs), against the oracle."""
    vocab, steps, L, n = 2048, 4, 640, 7
    w = S.make_weights(seed=27, num_layers=2, vocab_size=vocab, norm_std=0.1, max_seq_len=16)
    lens = [1, 2, 16, 17, 33, 250, 600]
    prompts = [S.make_prompt(Ln, seed=700 + i, vocab_size=vocab) for i, Ln in enumerate(lens)]
    eng = _engine(w, n, L, engine="gemm")
    dump = torch.zeros(n, steps, vocab, device="cuda")
    C.set_decode_attention(mma)
    C.set_logits_dump(dump)
    try:
        got = eng.generate_ids(prompts, steps)
    finally:
        C.set_logits_dump(None)
        C.set_decode_attention(1)
    worst = 0.0
    for b in range(n):
        want, logits = OracleDecoder(w, max_seq_len=L).generate_ids(prompts[b], steps, keep_logits=True)
        worst = max(worst, float((dump[b].cpu() - logits).abs().max()))
        assert got[b] == want, f"sequence {b} (prompt {lens[b]} tokens)"
    print(f"decode attention mma={mma}: worst max |logit - oracle| = {worst:.3e}")
    assert worst < LOGIT_TOL


def test_refusals(C):
    vocab = 2048
    w = S.make_weights(seed=1, num_layers=2, vocab_size=vocab, max_seq_len=16)
    eng = _engine(w, 6, 64, engine="gemm")
    with pytest.raises(ValueError):
        eng.generate_ids([[1]] * 7, 2)
    base = eng._base
    log = torch.zeros(4, dtype=torch.int32, device="cuda")
    common = (base._embed_weight, base._layer_weights_packed, base._final_norm_weight, base._lm_head_weight,
              base._cos_table, base._sin_table)
    with pytest.raises(RuntimeError, match="max_seq_len"):
        C.decode_batched([1, 2], [0, 63], 2, *common, eng._k_caches[:2], eng._v_caches[:2], [log, log.clone()],
                         base.num_layers, 64, base._attn_scale)
    with pytest.raises(RuntimeError, match="share"):
        C.decode_batched([1, 2], [0, 0], 2, *common, [eng._k_caches[0]] * 2, eng._v_caches[:2], [log, log.clone()],
                         base.num_layers, 64, base._attn_scale)
    assert len(eng.generate_ids([[1, 2, 3]] * 6, 3)[5]) == 3
