"""Continuous batching scheduler: host logic against a fake engine (CPU), and end to end on the GPU
against the single-sequence engine."""

import pytest
import torch

import synthetic as S
from scheduler import ContinuousBatcher


class FakeEngine:
    """Deterministic stand-in: the token after ``t`` at cache position ``p`` is ``(7 t + 3 p + 1) % 97``.
    Records what the scheduler asked for."""

    def __init__(self, num_sequences=4, max_seq_len=64):
        self.num_sequences, self.max_seq_len = num_sequences, max_seq_len
        self.positions = [0] * num_sequences
        self.launch_log = []

    @staticmethod
    def nxt(t, p):
        return (7 * t + 3 * p + 1) % 97

    def prefill_slot(self, b, ids):
        if any(t < 0 for t in ids):
            raise RuntimeError("bad token")
        self.positions[b] = len(ids)

    def decode_slots(self, slots, firsts, steps):
        self.launch_log.append((tuple(slots), steps))
        out = []
        for b, t in zip(slots, firsts):
            toks = []
            for _ in range(steps):
                t = self.nxt(t, self.positions[b])
                self.positions[b] += 1
                toks.append(t)
            out.append(toks)
        return out

    @classmethod
    def reference(cls, ids, n, eos=-1):
        t, p, out = ids[-1], len(ids) - 1, []
        for _ in range(n):
            t = cls.nxt(t, p)
            p += 1
            if t == eos:
                return out, "stop"
            out.append(t)
        return out, "length"


def test_every_request_matches_its_own_sequential_run():
    eng = FakeEngine(num_sequences=3)
    sch = ContinuousBatcher(eng, eos_token_id=None, quantum=5)
    reqs = [(S.make_prompt(1 + (i * 5) % 11, seed=i, vocab_size=97), 1 + (i * 7) % 23) for i in range(17)]
    futs = [sch.submit(ids, n) for ids, n in reqs]
    sch.run_until_idle()
    for (ids, n), f in zip(reqs, futs):
        r = f.result(timeout=0)
        want, why = FakeEngine.reference(ids, n)
        assert r.tokens == want and r.finish_reason == why == "length" and r.prompt_tokens == len(ids)
    assert sch.max_live == 3                                   # the slots were actually shared
    assert all(len(s) <= 3 and 1 <= q <= 5 for s, q in eng.launch_log)
    assert sch.launches == len(eng.launch_log) < sum(n for _, n in reqs)   # fewer launches than tokens
    # arrival order is admission order: request ids are handed out in submit order
    assert [f.result().rid for f in futs] == list(range(17))


def test_eos_frees_the_slot_and_is_not_returned():
    ids, n = [5, 9, 2], 30
    full, _ = FakeEngine.reference(ids, n)
    eos = full[4]
    eng = FakeEngine(num_sequences=2)
    sch = ContinuousBatcher(eng, eos_token_id=eos, quantum=3)
    f1 = sch.submit(ids, n)
    f2 = sch.submit([1, 2, 3, 4], 9)
    f3 = sch.submit([8], 4)                                    # waits for a slot
    sch.run_until_idle()
    want, why = FakeEngine.reference(ids, n, eos)
    assert why == "stop" and f1.result().tokens == want == full[:full.index(eos)]
    assert f1.result().finish_reason == "stop"
    for f, (i, k) in ((f2, ([1, 2, 3, 4], 9)), (f3, ([8], 4))):
        w, y = FakeEngine.reference(i, k, eos)
        assert f.result().tokens == w and f.result().finish_reason == y


def test_quantum_never_overruns_a_budget_and_bad_requests_fail_alone():
    eng = FakeEngine(num_sequences=2, max_seq_len=16)
    sch = ContinuousBatcher(eng, quantum=8)
    ok = sch.submit([3, 4], 3)
    too_long = sch.submit(list(range(10)), 10)                 # 9 + 10 > 16
    empty = sch.submit([], 4)
    zero = sch.submit([1, 2], 0)
    bad = sch.submit([5, -1, 7], 2)                            # the engine refuses the prompt
    later = sch.submit([6], 11)
    sch.run_until_idle()
    assert ok.result().tokens == FakeEngine.reference([3, 4], 3)[0]
    assert later.result().tokens == FakeEngine.reference([6], 11)[0]
    assert zero.result().tokens == []
    with pytest.raises(ValueError):
        too_long.result()
    with pytest.raises(ValueError):
        empty.result()
    with pytest.raises(RuntimeError):
        bad.result()
    # the first launch carried both live requests and stopped at the shorter budget
    assert eng.launch_log[0] == ((0, 1), 3)
    for b in range(2):
        assert eng.positions[b] <= 16


def test_background_thread_serves_submissions():
    eng = FakeEngine(num_sequences=4)
    sch = ContinuousBatcher(eng, quantum=4)
    sch.start()
    try:
        futs = [(ids, n, sch.submit(ids, n)) for ids, n in (([2, 3], 6), ([9], 13), ([4, 4, 4], 2))]
        for ids, n, f in futs:
            assert f.result(timeout=10).tokens == FakeEngine.reference(ids, n)[0]
    finally:
        sch.stop()


@pytest.mark.gpu
def test_gpu_continuous_batching_equals_single_sequence_engine(built_library, tiny_cfg):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from Model.Qwen06B_architecture import BatchDecoder, Decoder
    vocab = tiny_cfg["vocab_size"]
    w = S.weights_to(S.make_weights(seed=tiny_cfg["seed"], num_layers=tiny_cfg["num_layers"], vocab_size=vocab,
                                    norm_std=tiny_cfg["norm_std"], max_seq_len=16), "cuda")
    tok = S.StubTokenizer(-1, vocab)
    eng = BatchDecoder(weights=w, tokenizer=tok, num_sequences=4, max_seq_len=256, engine="persistent")
    reqs = [(S.make_prompt(3 + (i * 13) % 60, seed=100 + i, vocab_size=vocab), 4 + (i * 5) % 29) for i in range(11)]
    single = Decoder(weights=w, tokenizer=tok, verbose=False, max_seq_len=256)
    want = [single.generate_ids(ids, n) for ids, n in reqs]
    eos = want[2][3]                                           # a token that really occurs
    sch = ContinuousBatcher(eng, eos_token_id=eos, quantum=8)
    futs = [sch.submit(ids, n) for ids, n in reqs]
    sch.run_until_idle()
    for w_, f, (ids, n) in zip(want, futs, reqs):
        r = f.result(timeout=0)
        cut = w_[:w_.index(eos)] if eos in w_ else w_
        assert r.tokens == cut
        assert r.finish_reason == ("stop" if eos in w_ else "length")
    assert sch.max_live == 4 and sch.launches < sum(n for _, n in reqs)


def test_random_workloads_property():
    """Property test over random request mixes, slot counts, quanta and EOS ids: every request's answer equals
    its own sequential run, the slot limit holds, nobody overruns a budget, all futures resolve."""
    hypothesis = pytest.importorskip("hypothesis")
    from hypothesis import given, settings, strategies as st

    req = st.tuples(st.lists(st.integers(0, 96), min_size=1, max_size=12), st.integers(0, 40))

    @settings(max_examples=60, deadline=None)
    @given(reqs=st.lists(req, min_size=1, max_size=25), slots=st.integers(1, 9), quantum=st.integers(1, 17),
           eos=st.one_of(st.none(), st.integers(0, 96)))
    def run(reqs, slots, quantum, eos):
        eng = FakeEngine(num_sequences=slots, max_seq_len=64)
        sch = ContinuousBatcher(eng, eos_token_id=eos, quantum=quantum)
        futs = [sch.submit(ids, n) for ids, n in reqs]
        sch.run_until_idle()
        for (ids, n), f in zip(reqs, futs):
            r = f.result(timeout=0)
            want, why = FakeEngine.reference(ids, n, -1 if eos is None else eos) if n > 0 else ([], "length")
            assert r.tokens == want and r.finish_reason == why
        assert sch.max_live <= slots
        assert all(len(s) <= slots and len(set(s)) == len(s) and 1 <= q <= quantum for s, q in eng.launch_log)
        assert all(p <= 64 for p in eng.positions)

    run()


def test_overlapped_admission_gives_the_same_answers():
    """Prefill on its own thread: same tokens per request, slot limit respected, everything resolves; the fake
    engine's prefill sleeps so that decode rounds really run while a prefill is in flight."""
    import time

    class SlowPrefill(FakeEngine):
        def __init__(self, *a, **k):
            super().__init__(*a, **k)
            self.concurrent = 0

        def prefill_slot(self, b, ids):
            time.sleep(0.004)
            super().prefill_slot(b, ids)

        def decode_slots(self, slots, firsts, steps):
            time.sleep(0.001)
            return super().decode_slots(slots, firsts, steps)

    eng = SlowPrefill(num_sequences=3)
    sch = ContinuousBatcher(eng, eos_token_id=None, quantum=4, overlap_prefill=True)
    reqs = [(S.make_prompt(1 + (i * 5) % 11, seed=i, vocab_size=97), 2 + (i * 7) % 19) for i in range(14)]
    futs = [sch.submit(ids, n) for ids, n in reqs]
    sch.run_until_idle()
    sch.stop()
    for (ids, n), f in zip(reqs, futs):
        assert f.result(timeout=0).tokens == FakeEngine.reference(ids, n)[0]
    assert sch.max_live <= 3 and all(len(s) <= 3 for s, _ in eng.launch_log)
    # decode rounds with fewer than all slots live happened while later prefills were still running
    assert any(len(s) < 3 for s, _ in eng.launch_log[:5])


def test_live_limit_keeps_spare_slots_for_prefilled_requests():
    """With ``live_limit`` below the engine's slot count no launch carries more sequences than the limit; the other
    slots hold prefilled requests that take a seat as soon as one frees up, and every answer is still its own."""
    eng = FakeEngine(num_sequences=6)
    sch = ContinuousBatcher(eng, eos_token_id=None, quantum=4, live_limit=3)
    reqs = [(S.make_prompt(2 + (i * 3) % 7, seed=i, vocab_size=97), 3 + (i * 5) % 17) for i in range(14)]
    futs = [sch.submit(ids, n) for ids, n in reqs]
    sch.run_until_idle()
    sch.stop()
    for (ids, n), f in zip(reqs, futs):
        assert f.result(timeout=0).tokens == FakeEngine.reference(ids, n)[0]
    assert sch.max_live == 3 and all(len(s) <= 3 for s, _ in eng.launch_log)
    full = sum(1 for s, _ in eng.launch_log if len(s) == 3)
    assert full >= len(eng.launch_log) - 4        # seats are refilled at once: only the last rounds run short
    with pytest.raises(ValueError):
        ContinuousBatcher(eng, live_limit=0)


def test_waiting_requests_are_prefilled_together_when_the_engine_can():
    """An engine with ``prefill_slots`` gets every waiting request that fits its row budget in one call (prompts
    padded to multiples of 128 rows); a failing group falls back to one pass per request."""
    class Packing(FakeEngine):
        packed_prefill_rows = 512

        def __init__(self, **kw):
            super().__init__(**kw)
            self.groups = []

        def prefill_slots(self, slots, prompts):
            self.groups.append([len(p) for p in prompts])
            if any(t < 0 for p in prompts for t in p):
                raise RuntimeError("bad token")
            for b, p in zip(slots, prompts):
                self.positions[b] = len(p)

    eng = Packing(num_sequences=6, max_seq_len=400)
    sch = ContinuousBatcher(eng, eos_token_id=None, quantum=4)
    lens = [5, 130, 100, 300, 2, 7]            # rows 128 + 256 + 128 | 384 + 128 | 128
    reqs = [(S.make_prompt(n, seed=i, vocab_size=97), 6) for i, n in enumerate(lens)]
    reqs[4] = ([-3, 5], 6)                      # prompt_ids[:-1] holds a bad token: its group fails as a whole
    futs = [sch.submit(ids, n) for ids, n in reqs]
    sch.run_until_idle()
    sch.stop()
    assert eng.groups[0] == [4, 129, 99] and eng.groups[1] == [299, 1]
    for i, ((ids, n), f) in enumerate(zip(reqs, futs)):
        if i == 4:
            with pytest.raises(RuntimeError):
                f.result(timeout=0)
        else:
            assert f.result(timeout=0).tokens == FakeEngine.reference(ids, n)[0]


@pytest.mark.gpu
@pytest.mark.parametrize("table_rope", [False, True])
def test_gpu_packed_prefill_matches_one_prompt_per_pass(built_library, table_rope):
    """Several prompts through one tensor-core pass (``prefill_slots``): every slot's cache rows agree with a pass of
    its own to the rounding of a different GEMM tiling, and the tokens decoded from them are the same.  Also with
    the rotary angles read from the fp16 cos / sin tables."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import qwen_megakernel_C as C
    from Model.Qwen06B_architecture import BatchDecoder
    vocab = 2048
    w = S.weights_to(S.make_weights(seed=9, num_layers=3, vocab_size=vocab, norm_std=0.1, max_seq_len=16), "cuda")
    tok = S.StubTokenizer(-1, vocab)
    lens = [1, 37, 128, 129, 300, 700, 64, 1000]
    prompts = [S.make_prompt(n + 1, seed=300 + i, vocab_size=vocab) for i, n in enumerate(lens)]
    if table_rope:
        w = S.weights_to(S.make_weights(seed=9, num_layers=3, vocab_size=vocab, norm_std=0.1, max_seq_len=1100), "cuda")
    eng = BatchDecoder(weights=w, tokenizer=tok, num_sequences=len(lens), max_seq_len=1100, engine="gemm", prefill_mode="tensor",
                       rope_from_table=table_rope)
    try:
        _packed_against_single(eng, lens, prompts)
    finally:
        C.configure(rope_from_table=0)


def _packed_against_single(eng, lens, prompts):
    for b, ids in enumerate(prompts):
        eng.prefill_slot(b, ids[:-1])
    want_k = [eng._k_caches[b].clone() for b in range(len(lens))]
    want_v = [eng._v_caches[b].clone() for b in range(len(lens))]
    want = eng.decode_slots(list(range(len(lens))), [ids[-1] for ids in prompts], 12)
    for b in range(len(lens)):
        eng._k_caches[b].zero_()
        eng._v_caches[b].zero_()
    eng.prefill_slots(list(range(len(lens))), [ids[:-1] for ids in prompts])   # 128 + 128 + 128 + 256 + 384 + 768 + 128 + 1024 rows
    assert eng.positions == lens
    for b, n in enumerate(lens):
        got_k = eng._k_caches[b].view(3, 8, -1, 128)[:, :, :n].float()
        ref_k = want_k[b].view(3, 8, -1, 128)[:, :, :n].float()
        got_v = eng._v_caches[b].view(3, 8, -1, 128)[:, :, :n].float()
        ref_v = want_v[b].view(3, 8, -1, 128)[:, :, :n].float()
        assert (got_k - ref_k).abs().max().item() < 1e-2 and (got_v - ref_v).abs().max().item() < 1e-2   # fp16 operands, other tile shapes
        # rows past the prompt stay untouched
        assert eng._k_caches[b].view(3, 8, -1, 128)[:, :, n:].abs().max().item() == 0
    got = eng.decode_slots(list(range(len(lens))), [ids[-1] for ids in prompts], 12)
    assert got == want


@pytest.mark.gpu
def test_gpu_overlapped_prefill_matches_serial_scheduling(built_library, tiny_cfg):
    """Tensor-core engines, 8 slots: prefill of the next request on its own stream and thread while the live
    ones decode.  A sequence's tokens do not depend on who shares its launches, so both schedules must agree."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from Model.Qwen06B_architecture import BatchDecoder
    vocab = 2048
    w = S.weights_to(S.make_weights(seed=5, num_layers=2, vocab_size=vocab, norm_std=0.1, max_seq_len=16), "cuda")
    tok = S.StubTokenizer(-1, vocab)
    reqs = [(S.make_prompt(3 + (i * 37) % 300, seed=200 + i, vocab_size=vocab), 4 + (i * 5) % 23) for i in range(20)]
    outs = []
    for overlap in (False, True):
        eng = BatchDecoder(weights=w, tokenizer=tok, num_sequences=8, max_seq_len=384, engine="gemm", prefill_mode="tensor")
        assert eng.supports_overlap
        # (one prefill pass per request: with packed passes a cache's last bits depend on the group's GEMM tiling, and
        # the two schedules form different groups)
        sch = ContinuousBatcher(eng, eos_token_id=None, quantum=8, overlap_prefill=overlap, packed_prefill=False)
        futs = [sch.submit(ids, n) for ids, n in reqs]
        sch.run_until_idle()
        sch.stop()
        outs.append([f.result(timeout=0).tokens for f in futs])
        assert all(len(t) == n for t, (_, n) in zip(outs[-1], reqs))
    assert outs[0] == outs[1]
