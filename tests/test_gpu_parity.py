"""GPU parity tests: the sm_100a engine, called through the C-ABI op surface, against the CPU oracle.

Tolerances: greedy token IDs must be identical; logits within max-abs 3e-2 (the bound stated for
the fp16 engine); the asserts below also print the measured error, which is far smaller."""

import json
import os

import numpy as np
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


def _engine(cfg_or_weights, max_seq_len, tokenizer=None, **kw):
    from Model.Qwen06B_architecture import Decoder
    w = cfg_or_weights
    return Decoder(weights=S.weights_to(w, "cuda"), tokenizer=tokenizer, verbose=False, max_seq_len=max_seq_len, **kw)


def _tiny_weights(cfg):
    return S.make_weights(seed=cfg["seed"], num_layers=cfg["num_layers"], vocab_size=cfg["vocab_size"],
                          norm_std=cfg["norm_std"], max_seq_len=cfg["max_seq_len"])


def test_bounded_wait_reports_timeout(C):
    """A wait on a word nothing sets gives up after its budget and reports status 4; the context
    stays usable (no trap, no hang)."""
    assert C.selftest_wait_timeout(300) == 4
    assert torch.zeros(4, device="cuda").sum().item() == 0.0


def test_tiny_model_tokens_logits_and_cache(C, tiny_cfg):
    g = np.load(os.path.join(GOLDEN, "tiny_l2_v4096.npz"))
    w = _tiny_weights(tiny_cfg)
    ids = g["prompt"].tolist()
    eng = _engine(w, tiny_cfg["max_seq_len"], tokenizer=S.StubTokenizer(-1, tiny_cfg["vocab_size"]))
    steps = tiny_cfg["steps"]
    dump = torch.zeros(steps, tiny_cfg["vocab_size"], device="cuda")
    C.set_logits_dump(dump)
    try:
        toks = eng.generate_ids(ids, steps)
    finally:
        C.set_logits_dump(None)
    err = float((dump.cpu() - torch.from_numpy(g["logits"])).abs().max())
    print(f"tiny: max |logit - oracle| = {err:.3e}")
    assert toks == g["tokens"].tolist()
    assert err < LOGIT_TOL
    # KV rows against the oracle (fp16 storage: allow one ulp at |x| < 8)
    o = OracleDecoder(w, max_seq_len=tiny_cfg["max_seq_len"])
    o.generate_ids(ids, steps)
    n = len(ids) - 1 + steps
    assert (eng._k_cache[:, :, :n].float().cpu() - o.k_cache[:, :, :n].float()).abs().max() < 8e-3
    assert (eng._v_cache[:, :, :n].float().cpu() - o.v_cache[:, :, :n].float()).abs().max() < 8e-3
    assert eng.position == n
    # final-norm output buffer of the reference signature holds the last step's normalised state
    normed = eng._norm_out.cpu()
    assert (normed - o.last_normed).abs().max() < 1e-3


def test_step_prefill_and_generate_agree(C, tiny_cfg):
    """decode op, prefill op and generate op walk the same cache: three ways to the same tokens."""
    w = _tiny_weights(tiny_cfg)
    ids = S.make_prompt(9, seed=11, vocab_size=tiny_cfg["vocab_size"])
    eng = _engine(w, tiny_cfg["max_seq_len"], tokenizer=S.StubTokenizer(-1, tiny_cfg["vocab_size"]))
    ref = eng.generate_ids(ids, 6)
    eng.reset()
    cur = None
    for t in ids:
        cur = eng.step(t)          # token-serial through the single-step op
    got = [cur]
    for _ in range(5):
        got.append(eng.step(got[-1]))
    assert got == ref
    assert eng.position == len(ids) + 5
    text, n_in, n_out = eng.generate(" ".join(map(str, ids)), 6)
    assert (n_in, n_out) == (len(ids), 6) and text == " ".join(map(str, ref))


def test_eos_stops_and_is_trimmed(C, tiny_cfg):
    w = _tiny_weights(tiny_cfg)
    g = np.load(os.path.join(GOLDEN, "tiny_l2_v4096.npz"))
    ids, want = g["prompt"].tolist(), g["tokens"].tolist()
    stop = want[2]
    eng = _engine(w, tiny_cfg["max_seq_len"], tokenizer=S.StubTokenizer(stop, tiny_cfg["vocab_size"]))
    out = eng.generate_ids(ids, 8)
    assert out == want[:2]
    log = eng._output_log[:8].cpu().tolist()
    assert log[:3] == want[:3] and all(t == -1 for t in log[3:])   # EOS logged, rest untouched
    # the engine stays usable after an early stop
    eng.tokenizer = S.StubTokenizer(-1, tiny_cfg["vocab_size"])
    assert eng.generate_ids(ids, 8) == want


def test_table_rope_mode_matches_table_oracle(C, tiny_cfg):
    w = _tiny_weights(tiny_cfg)
    ids = S.make_prompt(10, seed=2, vocab_size=tiny_cfg["vocab_size"])
    o = OracleDecoder(w, max_seq_len=tiny_cfg["max_seq_len"], rope_from_tables=True)
    want, logits = o.generate_ids(ids, 4, keep_logits=True)
    eng = _engine(w, tiny_cfg["max_seq_len"], rope_from_table=True)
    dump = torch.zeros(4, tiny_cfg["vocab_size"], device="cuda")
    C.set_logits_dump(dump)
    try:
        got = eng.generate_ids(ids, 4)
    finally:
        C.set_logits_dump(None)
        C.configure(rope_from_table=0)
    assert got == want
    assert (dump.cpu() - logits).abs().max() < LOGIT_TOL


def test_split_kv_attention_long_context(C):
    """Context long enough that attention runs as several work items per kv head plus the merge."""
    cfg = dict(seed=4, num_layers=2, vocab_size=2048, norm_std=0.1, max_seq_len=1536)
    w = S.make_weights(seed=cfg["seed"], num_layers=2, vocab_size=2048, norm_std=0.1, max_seq_len=1536)
    ids = S.make_prompt(1400, seed=9, vocab_size=2048)
    o = OracleDecoder(w, max_seq_len=1536)
    want, logits = o.generate_ids(ids, 6, keep_logits=True)
    eng = _engine(w, 1536)
    dump = torch.zeros(6, 2048, device="cuda")
    C.set_logits_dump(dump)
    try:
        got = eng.generate_ids(ids, 6)
    finally:
        C.set_logits_dump(None)
    err = float((dump.cpu() - logits).abs().max())
    print(f"split-kv: max |logit - oracle| = {err:.3e}")
    assert got == want and err < LOGIT_TOL
    n = len(ids) - 1 + 6
    assert (eng._k_cache[:, :, :n].float().cpu() - o.k_cache[:, :, :n].float()).abs().max() < 8e-3


def test_context_beyond_2048_all_splits(C):
    """3000-token context: positions past the reference's 2048-row RoPE table, KV split over every
    available work item per head, uneven last split, chunks spanning several ring rounds."""
    w = S.make_weights(seed=6, num_layers=2, vocab_size=2048, norm_std=0.1, max_seq_len=16)
    ids = S.make_prompt(3000, seed=13, vocab_size=2048)
    o = OracleDecoder(w, max_seq_len=3072)
    want, logits = o.generate_ids(ids, 5, keep_logits=True)
    eng = _engine(w, 3072)
    dump = torch.zeros(5, 2048, device="cuda")
    C.set_logits_dump(dump)
    try:
        got = eng.generate_ids(ids, 5)
    finally:
        C.set_logits_dump(None)
    err = float((dump.cpu() - logits).abs().max())
    print(f"ctx 3000: max |logit - oracle| = {err:.3e}")
    assert got == want and err < LOGIT_TOL
    # 16 CTAs: two KV splits of ~1500 rows each, i.e. attention items of ~94 ring chunks on a 21-slot ring
    # (several laps inside one phase), and projection phases longer than the ring as well
    try:
        C.configure(max_ctas=16)
        eng2 = _engine(w, 3072)
        assert eng2.generate_ids(ids, 5) == want
    finally:
        C.configure(max_ctas=0)


def test_reduced_grid_gives_same_tokens(C, tiny_cfg):
    """A smaller persistent grid changes every CTA's row ranges and the number of KV splits; tokens and
    logits must not change beyond round-off."""
    g = np.load(os.path.join(GOLDEN, "tiny_l2_v4096.npz"))
    w = _tiny_weights(tiny_cfg)
    ids = g["prompt"].tolist()
    eng = _engine(w, tiny_cfg["max_seq_len"])
    try:
        for ctas in (8, 40, 97):
            C.configure(max_ctas=ctas)
            assert C.num_ctas() == ctas
            dump = torch.zeros(tiny_cfg["steps"], tiny_cfg["vocab_size"], device="cuda")
            C.set_logits_dump(dump)
            try:
                assert eng.generate_ids(ids, tiny_cfg["steps"]) == g["tokens"].tolist(), ctas
            finally:
                C.set_logits_dump(None)
            assert (dump.cpu() - torch.from_numpy(g["logits"])).abs().max() < LOGIT_TOL
    finally:
        C.configure(max_ctas=0)


def test_errors_are_reported_not_ignored(C, tiny_cfg):
    w = _tiny_weights(tiny_cfg)
    eng = _engine(w, tiny_cfg["max_seq_len"])
    ids = S.make_prompt(4, seed=1, vocab_size=tiny_cfg["vocab_size"])
    with pytest.raises(RuntimeError, match="max_seq_len"):
        eng.generate_ids(ids, tiny_cfg["max_seq_len"])   # 3 prompt rows + 64 steps > 64
    with pytest.raises(RuntimeError, match="int32"):
        eng._gen(1, 2, *eng._common(), torch.zeros(4, device="cuda"), eng.num_layers, 0, eng.max_seq_len, 0.1)
    with pytest.raises(RuntimeError, match="numel"):
        eng._gen(1, 8, *eng._common(), torch.zeros(4, dtype=torch.int32, device="cuda"), eng.num_layers, 0,
                 eng.max_seq_len, 0.1)
    with pytest.raises(RuntimeError, match="vocab"):
        eng.prefill_ids([1, tiny_cfg["vocab_size"] + 5])
    # still healthy
    eng.reset()
    assert len(eng.generate_ids(ids, 3)) == 3


def test_full_model_32_greedy_steps_match_oracle(C, full_cfg):
    """The headline parity case: Qwen3-0.6B shape, seed 0, 32-token prompt, 32 greedy steps.
    Token IDs identical to the oracle's (golden file, re-derived here on the CPU), logits within 3e-2."""
    g = json.load(open(os.path.join(GOLDEN, "full_seed0_prompt32.json")))
    w = S.make_weights(seed=full_cfg["seed"], num_layers=28, vocab_size=S.VOCAB_SIZE, max_seq_len=128)
    ids = g["prompt"]
    o = OracleDecoder(w, max_seq_len=128)
    want, logits = o.generate_ids(ids, 32, keep_logits=True)
    assert want == g["tokens"], "oracle no longer reproduces its own golden tokens"
    eng = _engine(w, 128)
    dump = torch.zeros(32, S.VOCAB_SIZE, device="cuda")
    C.set_logits_dump(dump)
    try:
        got = eng.generate_ids(ids, 32)
    finally:
        C.set_logits_dump(None)
    err = float((dump.cpu() - logits).abs().max())
    print(f"full: max |logit - oracle| = {err:.3e}; min greedy margin = {g['min_margin']:.3e}")
    assert got == want
    assert err < LOGIT_TOL
    # run twice: bit-identical logits (fixed summation order everywhere)
    dump2 = torch.zeros(32, S.VOCAB_SIZE, device="cuda")
    C.set_logits_dump(dump2)
    try:
        assert eng.generate_ids(ids, 32) == want
    finally:
        C.set_logits_dump(None)
    assert torch.equal(dump, dump2)


def _golden_ctx4096():
    return json.load(open(os.path.join(GOLDEN, "full_seed0_prompt4096.json")))


@pytest.mark.parametrize("prefill_mode", ["serial", "tensor"])
def test_benchmark_configuration_matches_golden(C, prefill_mode):
    """The configuration bench.py times (full model, seed 0, make_prompt(4096, seed 0), max_seq_len 4352):
    first 8 greedy tokens identical to the oracle's golden file, their top-8 logits within 3e-2.  Both prefill
    paths: the token-serial op (fp32 activations) and the chunked tensor-core prefill (fp16 GEMM operands)."""
    g = _golden_ctx4096()
    cfg = g["config"]
    ids = S.make_prompt(cfg["prompt_len"], seed=cfg["prompt_seed"])
    assert ids[:8] == g["prompt_head"] and ids[-8:] == g["prompt_tail"]
    w = S.make_weights(seed=cfg["seed"], num_layers=cfg["num_layers"], vocab_size=cfg["vocab_size"], max_seq_len=16)
    eng = _engine(w, cfg["max_seq_len"], prefill_mode=prefill_mode)
    steps = cfg["steps"]
    dump = torch.zeros(steps, cfg["vocab_size"], device="cuda")
    C.set_logits_dump(dump)
    try:
        got = eng.generate_ids(ids, steps)
    finally:
        C.set_logits_dump(None)
    idx = torch.tensor(g["top8_indices"], device="cuda")
    vals = torch.gather(dump, 1, idx).cpu()
    err = float((vals - torch.tensor(g["top8_values"])).abs().max())
    print(f"ctx 4096 ({prefill_mode} prefill): max |top-8 logit - golden| = {err:.3e}; min margin {g['min_margin']:.3e}")
    assert got == g["tokens"]
    assert err < LOGIT_TOL


def test_fused_and_unfused_kernels_agree(C, tiny_cfg):
    """The fused kernels (split-K O/down slices, integer all-reduced residual sums; 2 = row products on the tensor
    cores with the activations split into two fp16 columns, 1 = on the CUDA cores) and the unfused kernel (0) sum in
    different orders: same tokens, logits equal to round-off, and each bit-identical to itself run to run."""
    g = np.load(os.path.join(GOLDEN, "tiny_l2_v4096.npz"))
    w = _tiny_weights(tiny_cfg)
    ids = g["prompt"].tolist()
    eng = _engine(w, tiny_cfg["max_seq_len"])
    dumps = {}
    try:
        for mode in (2, 1, 0, 2, 1):
            C.set_fused(fused=mode)
            dump = torch.zeros(tiny_cfg["steps"], tiny_cfg["vocab_size"], device="cuda")
            C.set_logits_dump(dump)
            try:
                assert eng.generate_ids(ids, tiny_cfg["steps"]) == g["tokens"].tolist(), mode
            finally:
                C.set_logits_dump(None)
            assert (dump.cpu() - torch.from_numpy(g["logits"])).abs().max() < LOGIT_TOL
            if mode in dumps:
                assert torch.equal(dumps[mode], dump), "fused kernel is not reproducible run to run"
            dumps[mode] = dump
        for a, b in ((0, 1), (0, 2)):
            diff = float((dumps[a] - dumps[b]).abs().max())
            print(f"kernel {a} vs kernel {b}: max |logit diff| = {diff:.3e}")
            assert diff < 1e-3
        # two accumulator copies per sum: same integers, added in two groups
        for mode in (1, 2):
            C.set_fused(fused=mode, red_copies=2)
            dump = torch.zeros(tiny_cfg["steps"], tiny_cfg["vocab_size"], device="cuda")
            C.set_logits_dump(dump)
            try:
                assert eng.generate_ids(ids, tiny_cfg["steps"]) == g["tokens"].tolist()
            finally:
                C.set_logits_dump(None)
            assert torch.equal(dump, dumps[mode]), "integer sums must not depend on how contributions are grouped"
    finally:
        C.set_fused(fused=2, red_copies=1)


def test_kmajor_copies_follow_the_weights(C, tiny_cfg):
    """The fused kernel reads library-made K-major copies of W_o / W_down.  New weights behind the SAME layer
    table (same addresses, new contents) must be picked up by the per-call hash check."""
    w1 = _tiny_weights(tiny_cfg)
    cfg2 = dict(tiny_cfg, seed=tiny_cfg["seed"] + 1)
    w2 = _tiny_weights(cfg2)
    ids = S.make_prompt(10, seed=4, vocab_size=tiny_cfg["vocab_size"])
    want1 = OracleDecoder(w1, max_seq_len=tiny_cfg["max_seq_len"]).generate_ids(ids, 5)[0]
    want2 = OracleDecoder(w2, max_seq_len=tiny_cfg["max_seq_len"]).generate_ids(ids, 5)[0]
    assert want1 != want2
    dev = S.weights_to(w1, "cuda")
    from Model.Qwen06B_architecture import Decoder
    eng = Decoder(weights=dev, verbose=False, max_seq_len=tiny_cfg["max_seq_len"])
    assert eng.generate_ids(ids, 5) == want1
    for dst, src in zip(dev["layer_weights"], w2["layer_weights"]):     # overwrite in place: the table is unchanged
        dst.copy_(src)
    dev["embed_weight"].copy_(w2["embed_weight"])
    dev["final_norm_weight"].copy_(w2["final_norm_weight"])
    assert eng.generate_ids(ids, 5) == want2


def test_decoders_with_different_options_share_a_gpu(C, tiny_cfg):
    """Vocabulary size, weight format and RoPE mode are per-device state of the library; every decoder re-applies
    its own before each op, so two live decoders that differ in them can be used in turn."""
    import quantize
    w_a = _tiny_weights(tiny_cfg)
    cfg_b = dict(tiny_cfg, seed=tiny_cfg["seed"] + 7, vocab_size=2048)
    w_b = _tiny_weights(cfg_b)
    ids_a = S.make_prompt(9, seed=21, vocab_size=tiny_cfg["vocab_size"])
    ids_b = S.make_prompt(7, seed=22, vocab_size=cfg_b["vocab_size"])
    eng_b_w, oracle_b_w = quantize.quantize_weights_fp8(w_b)
    want_a = OracleDecoder(w_a, max_seq_len=tiny_cfg["max_seq_len"]).generate_ids(ids_a, 5)[0]
    want_b = OracleDecoder(oracle_b_w, max_seq_len=tiny_cfg["max_seq_len"]).generate_ids(ids_b, 5)[0]
    from Model.Qwen06B_architecture import Decoder
    a = Decoder(weights=S.weights_to(w_a, "cuda"), verbose=False, max_seq_len=tiny_cfg["max_seq_len"])
    b = Decoder(weights=S.weights_to(eng_b_w, "cuda"), verbose=False, max_seq_len=tiny_cfg["max_seq_len"],
                weight_format="fp8")
    try:
        for _ in range(2):
            assert a.generate_ids(ids_a, 5) == want_a
            assert b.generate_ids(ids_b, 5) == want_b
        # step mode too
        a.reset()
        b.reset()
        ta = tb = None
        for t in ids_a:
            ta = a.step(t)
        for t in ids_b:
            tb = b.step(t)
        assert ta == want_a[0] and tb == want_b[0]
        with pytest.raises(RuntimeError, match="weight_format"):
            Decoder(weights=S.weights_to(eng_b_w, "cuda"), verbose=False, max_seq_len=tiny_cfg["max_seq_len"])
    finally:
        C.set_weight_format("fp16")
        C.configure(vocab_size=tiny_cfg["vocab_size"])


def test_engine_handles_from_two_threads(C, tiny_cfg):
    """Engine handles (``qmk_engine_create``): each carries one client's options and applies them with the op under
    one hold of the library's lock, so two threads that decode with different vocabularies and weight formats on one
    GPU - with no re-application by the caller - both get the oracle's tokens.  Destroying a handle frees the K-major
    weight copies made for its table; the decoder that owned it can no longer be used."""
    import threading
    import quantize
    from Model.Qwen06B_architecture import Decoder
    w_a = _tiny_weights(tiny_cfg)
    cfg_b = dict(tiny_cfg, seed=tiny_cfg["seed"] + 11, vocab_size=2048)
    eng_b_w, oracle_b_w = quantize.quantize_weights_fp8(_tiny_weights(cfg_b))
    ids_a = S.make_prompt(9, seed=31, vocab_size=tiny_cfg["vocab_size"])
    ids_b = S.make_prompt(7, seed=32, vocab_size=cfg_b["vocab_size"])
    want_a = OracleDecoder(w_a, max_seq_len=tiny_cfg["max_seq_len"]).generate_ids(ids_a, 5)[0]
    want_b = OracleDecoder(oracle_b_w, max_seq_len=tiny_cfg["max_seq_len"]).generate_ids(ids_b, 5)[0]
    a = Decoder(weights=S.weights_to(w_a, "cuda"), verbose=False, max_seq_len=tiny_cfg["max_seq_len"])
    b = Decoder(weights=S.weights_to(eng_b_w, "cuda"), verbose=False, max_seq_len=tiny_cfg["max_seq_len"],
                weight_format="fp8")
    assert a._engine is not None and b._engine is not None
    results, errors = {"a": [], "b": []}, []

    def work(name, dec, ids):
        try:
            torch.cuda.set_device(0)
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                for _ in range(6):
                    results[name].append(dec.generate_ids(ids, 5))
        except Exception as exc:   # surfaced below: an exception in a thread would otherwise pass silently
            errors.append(repr(exc))

    try:
        torch.cuda.synchronize()
        threads = [threading.Thread(target=work, args=("a", a, ids_a)), threading.Thread(target=work, args=("b", b, ids_b))]
        for t in threads:
            t.start()
        for t in threads:
            t.join(timeout=300)
        assert not errors, errors
        assert results["a"] == [want_a] * 6 and results["b"] == [want_b] * 6
        # bad configurations are refused without a handle
        with pytest.raises(RuntimeError, match="qmk_engine_create"):
            C.Engine(vocab_size=2048, weight_format="fp16", fused=7)
        a._engine.close()
        with pytest.raises(RuntimeError, match="after close"):
            a.generate_ids(ids_a, 2)
        assert b.generate_ids(ids_b, 5) == want_b
    finally:
        C.set_weight_format("fp16")
        C.configure(vocab_size=tiny_cfg["vocab_size"])
