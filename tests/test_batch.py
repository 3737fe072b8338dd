"""GPU parity of the multi-sequence launch (``generate_batch`` / ``BatchDecoder``) against the CPU oracle.

Every sequence of a launch is checked on its own against the oracle run on the same prompt: identical
greedy token IDs, logits within 3e-2 max-abs (the bound stated for the fp16 engine).  Sequences differ
in length on purpose, so that each one has its own position, RoPE angles and attention split."""

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


def _batch_engine(w, n, max_seq_len, **kw):
    from Model.Qwen06B_architecture import BatchDecoder
    kw.setdefault("engine", "persistent")   # this file covers the multi-sequence persistent kernel
    return BatchDecoder(weights=S.weights_to(w, "cuda"), tokenizer=S.StubTokenizer(-1, w["embed_weight"].shape[0]),
                        num_sequences=n, max_seq_len=max_seq_len, **kw)


def _oracle(w, max_seq_len, prompts, steps):
    want, logits = [], []
    for ids in prompts:
        t, lg = OracleDecoder(w, max_seq_len=max_seq_len).generate_ids(ids, steps, keep_logits=True)
        want.append(t)
        logits.append(lg)
    return want, logits


def _run_with_dump(C, eng, prompts, steps, vocab):
    dump = torch.zeros(len(prompts), steps, vocab, device="cuda")
    C.set_logits_dump(dump)
    try:
        got = eng.generate_ids(prompts, steps)
    finally:
        C.set_logits_dump(None)
    return got, dump.cpu()


@pytest.mark.parametrize("n", [1, 2, 3, 4])
def test_tiny_model_every_group_width(C, tiny_cfg, n):
    """1, 2, 3 and 4 sequences per launch (12, 6, 4 and 3 math warps per sequence)."""
    w = S.make_weights(seed=tiny_cfg["seed"], num_layers=tiny_cfg["num_layers"], vocab_size=tiny_cfg["vocab_size"],
                       norm_std=tiny_cfg["norm_std"], max_seq_len=tiny_cfg["max_seq_len"])
    lens = [12, 5, 23, 1][:n]
    prompts = [S.make_prompt(L, seed=20 + i, vocab_size=tiny_cfg["vocab_size"]) for i, L in enumerate(lens)]
    steps = 7
    want, logits = _oracle(w, tiny_cfg["max_seq_len"], prompts, steps)
    eng = _batch_engine(w, n, tiny_cfg["max_seq_len"])
    got, dump = _run_with_dump(C, eng, prompts, steps, tiny_cfg["vocab_size"])
    for b in range(n):
        err = float((dump[b] - logits[b]).abs().max())
        print(f"batch {n}, sequence {b}: max |logit - oracle| = {err:.3e}")
        assert got[b] == want[b]
        assert err < LOGIT_TOL
    assert eng.positions[:n] == [L - 1 + steps for L in lens]
    # second call on the same engine: caches are reused from position 0, same answer
    assert eng.generate_ids(prompts, steps) == want


def test_mixed_context_lengths_split_and_unsplit(C):
    """One launch with a 1400-token context (attention split over several CTAs + merge), a 700-token
    one and two short ones: the per-sequence split counts and ring chunk counts all differ."""
    w = S.make_weights(seed=4, num_layers=2, vocab_size=2048, norm_std=0.1, max_seq_len=16)
    lens = [1400, 3, 700, 130]
    prompts = [S.make_prompt(L, seed=40 + i, vocab_size=2048) for i, L in enumerate(lens)]
    steps = 5
    want, logits = _oracle(w, 1536, prompts, steps)
    eng = _batch_engine(w, 4, 1536)
    got, dump = _run_with_dump(C, eng, prompts, steps, 2048)
    for b in range(4):
        err = float((dump[b] - logits[b]).abs().max())
        print(f"mixed contexts, sequence {b} (len {lens[b]}): max |logit - oracle| = {err:.3e}")
        assert got[b] == want[b]
        assert err < LOGIT_TOL
    # cache rows of the long sequence against the oracle's (fp16 storage)
    o = OracleDecoder(w, max_seq_len=1536)
    o.generate_ids(prompts[0], steps)
    n = lens[0] - 1 + steps
    assert (eng._k_caches[0][:, :, :n].float().cpu() - o.k_cache[:, :, :n].float()).abs().max() < 8e-3
    assert (eng._v_caches[0][:, :, :n].float().cpu() - o.v_cache[:, :, :n].float()).abs().max() < 8e-3


def test_long_contexts_jump_several_ring_laps(C):
    """Four contexts above 2000 tokens: every sequence's attention item brings about nine cache chunks
    into the 13-slot ring, so the later groups jump more than two ring laps ahead when they skip the
    other sequences' chunks (the case the issued-chunk check in front of the parity wait exists for)."""
    w = S.make_weights(seed=8, num_layers=2, vocab_size=2048, norm_std=0.1, max_seq_len=16)
    lens = [2300, 2200, 2100, 2050]
    prompts = [S.make_prompt(L, seed=80 + i, vocab_size=2048) for i, L in enumerate(lens)]
    steps = 4
    want, logits = _oracle(w, 2560, prompts, steps)
    eng = _batch_engine(w, 4, 2560)
    got, dump = _run_with_dump(C, eng, prompts, steps, 2048)
    for b in range(4):
        err = float((dump[b] - logits[b]).abs().max())
        print(f"long contexts, sequence {b} (len {lens[b]}): max |logit - oracle| = {err:.3e}")
        assert got[b] == want[b]
        assert err < LOGIT_TOL
    eng2 = _batch_engine(w, 2, 2560)
    assert eng2.generate_ids(prompts[:2], steps) == want[:2]


def test_full_model_four_sequences_match_single_sequence_and_golden(C, full_cfg):
    """Qwen3-0.6B shape.  Sequence 0 is the golden prompt (token IDs from the committed oracle run);
    all four must equal what the single-sequence engine produces for the same prompts."""
    from Model.Qwen06B_architecture import Decoder
    g = json.load(open(os.path.join(GOLDEN, "full_seed0_prompt32.json")))
    w = S.make_weights(seed=full_cfg["seed"], num_layers=28, vocab_size=S.VOCAB_SIZE, max_seq_len=128)
    prompts = [g["prompt"]] + [S.make_prompt(L, seed=60 + i) for i, L in enumerate([7, 50, 19])]
    steps = 32
    eng = _batch_engine(w, 4, 128)
    got = eng.generate_ids(prompts, steps)
    assert got[0] == g["tokens"]
    single = Decoder(weights=eng._base._weights, tokenizer=S.StubTokenizer(-1), verbose=False, max_seq_len=128)
    for b in range(4):
        assert got[b] == single.generate_ids(prompts[b], steps), f"sequence {b}"
    # deterministic: the same launch twice gives the same tokens
    assert eng.generate_ids(prompts, steps) == got


def test_eos_is_cut_on_the_host(C, tiny_cfg):
    w = S.make_weights(seed=tiny_cfg["seed"], num_layers=tiny_cfg["num_layers"], vocab_size=tiny_cfg["vocab_size"],
                       norm_std=tiny_cfg["norm_std"], max_seq_len=tiny_cfg["max_seq_len"])
    prompts = [S.make_prompt(L, seed=20 + i, vocab_size=tiny_cfg["vocab_size"]) for i, L in enumerate([12, 5])]
    eng = _batch_engine(w, 2, tiny_cfg["max_seq_len"])
    full = eng.generate_ids(prompts, 8)
    stop = full[0][3]
    eng.tokenizer = eng._base.tokenizer = S.StubTokenizer(stop, tiny_cfg["vocab_size"])
    cut = eng.generate_ids(prompts, 8)
    for b in range(2):
        want = full[b][:full[b].index(stop)] if stop in full[b] else full[b]
        assert cut[b] == want


def test_bad_arguments_are_refused(C, tiny_cfg):
    w = S.make_weights(seed=1, num_layers=2, vocab_size=tiny_cfg["vocab_size"], max_seq_len=64)
    eng = _batch_engine(w, 2, 64)
    base = eng._base
    log = torch.zeros(4, dtype=torch.int32, device="cuda")
    common = (base._embed_weight, base._layer_weights_packed, base._final_norm_weight, base._lm_head_weight,
              base._cos_table, base._sin_table)
    with pytest.raises(RuntimeError, match="share"):   # same cache twice
        C.generate_batch([1, 2], [0, 0], 2, *common, [eng._k_caches[0]] * 2, eng._v_caches[:2], [log, log.clone()],
                         base.num_layers, 64, base._attn_scale)
    with pytest.raises(RuntimeError, match="max_seq_len"):   # one sequence would run past its cache
        C.generate_batch([1, 2], [0, 63], 2, *common, eng._k_caches[:2], eng._v_caches[:2], [log, log.clone()],
                         base.num_layers, 64, base._attn_scale)
    with pytest.raises(RuntimeError, match="1 to 4"):
        C.generate_batch([1] * 5, [0] * 5, 2, *common, eng._k_caches[:1] * 5, eng._v_caches[:1] * 5, [log] * 5,
                         base.num_layers, 64, base._attn_scale)
    # still healthy
    assert len(eng.generate_ids([[1, 2, 3], [4, 5]], 3)[0]) == 3
