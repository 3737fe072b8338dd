"""CPU tests of the oracle: pinned against its golden files, cross-checked against an independent
implementation (transformers' Qwen3), and checked for internal consistency."""

import json
import os

import numpy as np
import pytest
import torch

import synthetic as S
from oracle.decoder_ref import Decoder

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _tiny(cfg, **kw):
    w = S.make_weights(seed=cfg["seed"], num_layers=cfg["num_layers"], vocab_size=cfg["vocab_size"],
                       norm_std=cfg["norm_std"], max_seq_len=cfg["max_seq_len"])
    ids = S.make_prompt(cfg["prompt_len"], seed=cfg["prompt_seed"], vocab_size=cfg["vocab_size"])
    return w, ids, Decoder(w, max_seq_len=cfg["max_seq_len"], **kw)


def test_synthetic_is_deterministic():
    a = S.make_weights(seed=7, num_layers=1, vocab_size=512)
    b = S.make_weights(seed=7, num_layers=1, vocab_size=512)
    assert torch.equal(a["embed_weight"], b["embed_weight"])
    assert all(torch.equal(x, y) for x, y in zip(a["layer_weights"], b["layer_weights"]))
    assert a["lm_head_weight"] is a["embed_weight"]
    assert len(a["layer_weights"]) == 11
    assert [tuple(t.shape) for t in a["layer_weights"]] == [s for _, s in S.LAYER_FIELDS]
    assert S.make_prompt(5, seed=1) == S.make_prompt(5, seed=1)
    assert S.weight_bytes_fp16() == 1_192_101_888
    assert S.decode_step_bytes(1) - S.weight_bytes_fp16() == 2 * 28 * 4096


def test_tiny_golden_reproduced(tiny_cfg):
    g = np.load(os.path.join(GOLDEN, "tiny_l2_v4096.npz"))
    w, ids, d = _tiny(tiny_cfg)
    assert ids == g["prompt"].tolist()
    d.prefill(ids[:-1])
    cur, toks = ids[-1], []
    for s in range(tiny_cfg["steps"]):
        cur = d.step(cur, trace=(s == 0))
        if s == 0:
            for li, tr in d.trace.items():
                for k, v in tr.items():
                    np.testing.assert_allclose(v[0].numpy(), g[f"l{li}_{k}"], rtol=0, atol=2e-5)
        np.testing.assert_allclose(d.last_logits.numpy(), g["logits"][s], rtol=0, atol=5e-5)
        toks.append(cur)
    assert toks == g["tokens"].tolist()


def test_serial_equals_batched_prefill(tiny_cfg):
    w, ids, d = _tiny(tiny_cfg, kv_dtype=torch.float32)   # fp32 cache: no rounding flips between the two orders
    for t in ids:
        d.step(t)
    serial_logits, serial_k = d.last_logits.clone(), d.k_cache.clone()
    d.reset()
    d.prefill(ids[:-1], chunk=5)
    d.step(ids[-1])
    assert (serial_logits - d.last_logits).abs().max() < 2e-5
    assert (serial_k - d.k_cache).abs().max() < 2e-5


def test_generate_api_and_eos(tiny_cfg):
    w, ids, d = _tiny(tiny_cfg)
    toks, _ = d.generate_ids(ids, 8)
    g = np.load(os.path.join(GOLDEN, "tiny_l2_v4096.npz"))
    assert toks == g["tokens"].tolist()
    stop = toks[2]
    toks2, _ = d.generate_ids(ids, 8, eos_token_id=stop)
    assert toks2 == toks[:toks.index(stop)]
    d.tokenizer = S.StubTokenizer(eos_token_id=-1, vocab_size=tiny_cfg["vocab_size"])
    text, n_in, n_out = d.generate(" ".join(map(str, ids)), 4)
    assert (n_in, n_out) == (len(ids), 4) and text == " ".join(map(str, toks[:4]))


def test_against_transformers_qwen3(tiny_cfg):
    """Independent implementation, same weights: logits agree to fp32 round-off."""
    tr = pytest.importorskip("transformers")
    w, ids, d = _tiny(tiny_cfg, kv_dtype=torch.float32)
    cfg = tr.Qwen3Config(hidden_size=1024, num_hidden_layers=tiny_cfg["num_layers"], num_attention_heads=16,
                         num_key_value_heads=8, head_dim=128, intermediate_size=3072,
                         vocab_size=tiny_cfg["vocab_size"], rms_norm_eps=1e-6, tie_word_embeddings=True,
                         rope_parameters={"rope_theta": 1e6, "rope_type": "default"}, max_position_embeddings=64)
    m = tr.Qwen3ForCausalLM(cfg).float().eval()
    names = ["input_layernorm", "self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.q_norm",
             "self_attn.k_norm", "self_attn.o_proj", "post_attention_layernorm", "mlp.gate_proj", "mlp.up_proj",
             "mlp.down_proj"]
    sd = {f"model.layers.{li}.{n}.weight": w["layer_weights"][li * 11 + j].float()
          for li in range(tiny_cfg["num_layers"]) for j, n in enumerate(names)}
    sd["model.embed_tokens.weight"] = w["embed_weight"].float()
    sd["model.norm.weight"] = w["final_norm_weight"].float()
    sd["lm_head.weight"] = w["embed_weight"].float()
    missing = m.load_state_dict(sd, strict=False)
    assert not missing.missing_keys and not missing.unexpected_keys
    with torch.no_grad():
        hf = m(torch.tensor([ids])).logits[0]
    d.prefill(ids[:-1])
    d.step(ids[-1])
    assert (hf[-1] - d.last_logits).abs().max() < 2e-5


def test_against_transformers_qwen3_full_depth():
    """The same cross-check on the benchmarked shape: 28 layers, vocabulary 151936, seed-0 weights, the first 12
    tokens of the 32-token golden prompt.  Also ties the golden file to the independent implementation: at the
    12th position both predict from the same logits."""
    tr = pytest.importorskip("transformers")
    w = S.make_weights(seed=0, max_seq_len=16)
    ids = S.make_prompt(32, seed=0)[:12]
    d = Decoder(w, max_seq_len=16, kv_dtype=torch.float32)
    cfg = tr.Qwen3Config(hidden_size=1024, num_hidden_layers=S.NUM_LAYERS, num_attention_heads=16, num_key_value_heads=8,
                         head_dim=128, intermediate_size=3072, vocab_size=S.VOCAB_SIZE, rms_norm_eps=1e-6,
                         tie_word_embeddings=True, rope_parameters={"rope_theta": 1e6, "rope_type": "default"},
                         max_position_embeddings=64)
    m = tr.Qwen3ForCausalLM(cfg).float().eval()
    names = ["input_layernorm", "self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.q_norm",
             "self_attn.k_norm", "self_attn.o_proj", "post_attention_layernorm", "mlp.gate_proj", "mlp.up_proj",
             "mlp.down_proj"]
    sd = {f"model.layers.{li}.{n}.weight": w["layer_weights"][li * 11 + j].float()
          for li in range(S.NUM_LAYERS) for j, n in enumerate(names)}
    sd["model.embed_tokens.weight"] = w["embed_weight"].float()
    sd["model.norm.weight"] = w["final_norm_weight"].float()
    sd["lm_head.weight"] = w["embed_weight"].float()
    missing = m.load_state_dict(sd, strict=False)
    assert not missing.missing_keys and not missing.unexpected_keys
    with torch.no_grad():
        hf = m(torch.tensor([ids])).logits[0]
    d.prefill(ids[:-1])
    tok = d.step(ids[-1])
    err = float((hf[-1] - d.last_logits).abs().max())
    print(f"28 layers: max |oracle - transformers| = {err:.3e}")
    assert err < 5e-5
    assert tok == int(torch.argmax(hf[-1]))


def test_benchmark_golden_file_is_consistent():
    g = json.load(open(os.path.join(GOLDEN, "full_seed0_prompt4096.json")))
    ids = S.make_prompt(g["config"]["prompt_len"], seed=g["config"]["prompt_seed"])
    assert ids[:8] == g["prompt_head"] and ids[-8:] == g["prompt_tail"] and len(ids) == g["prompt_len"] == 4096
    assert len(g["tokens"]) == 8 and [r[0] for r in g["top8_indices"]] == g["tokens"]
    assert g["min_margin"] == min(g["margins"]) > 0.1


def test_full_golden_file_is_consistent():
    """Cheap checks of the full-size golden file (the full-size oracle run itself is exercised by the
    GPU parity test and by make_golden.py)."""
    g = json.load(open(os.path.join(GOLDEN, "full_seed0_prompt32.json")))
    assert g["prompt"] == S.make_prompt(32, seed=0)
    assert len(g["tokens"]) == 32 and all(0 <= t < S.VOCAB_SIZE for t in g["tokens"])
    assert [r[0] for r in g["top8_indices"]] == g["tokens"]
    assert g["min_margin"] == min(g["margins"]) > 0
    assert g["fp32_kv_tokens"] == g["tokens"]
