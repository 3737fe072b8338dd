"""``load_weights`` on a checkpoint written by transformers itself: a randomly initialised Qwen3 model of the real
layer shapes (two layers, small vocabulary) saved with ``save_pretrained`` next to a word-level tokenizer.  No
Qwen3-0.6B checkpoint is available offline; what is checked is the mapping from the checkpoint's tensor names to the
reference layout (11 tensors per layer in table order, tied LM head, fp16, rotary tables) and that a decoder built
from the loaded dictionary reproduces the transformers model's logits."""

import os
import sys

import pytest
import torch

import synthetic as S
from oracle.decoder_ref import Decoder as OracleDecoder

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "qwen3-0.6b-megakernel-rtx-5090_b200"))

VOCAB, LAYERS, MAX_LEN = 512, 2, 64


@pytest.fixture(scope="module")
def checkpoint(tmp_path_factory):
    tr = pytest.importorskip("transformers")
    tk = pytest.importorskip("tokenizers")
    path = str(tmp_path_factory.mktemp("qwen3_tiny"))
    torch.manual_seed(11)
    cfg = tr.Qwen3Config(hidden_size=1024, num_hidden_layers=LAYERS, num_attention_heads=16, num_key_value_heads=8,
                         head_dim=128, intermediate_size=3072, vocab_size=VOCAB, rms_norm_eps=1e-6,
                         tie_word_embeddings=True, rope_parameters={"rope_theta": 1e6, "rope_type": "default"},
                         max_position_embeddings=MAX_LEN)
    model = tr.Qwen3ForCausalLM(cfg).to(torch.float16)
    with torch.no_grad():            # norm weights away from 1 so that a swapped pair of norms would show
        for name, p in model.named_parameters():
            if "norm" in name:
                p.copy_((1.0 + 0.1 * torch.randn_like(p.float())).to(torch.float16))
    model.save_pretrained(path)
    vocab = {str(i): i for i in range(VOCAB - 1)}
    vocab["<unk>"] = VOCAB - 1
    tok = tk.Tokenizer(tk.models.WordLevel(vocab=vocab, unk_token="<unk>"))
    tok.pre_tokenizer = tk.pre_tokenizers.WhitespaceSplit()
    tr.PreTrainedTokenizerFast(tokenizer_object=tok, unk_token="<unk>").save_pretrained(path)
    # the comparison model is read back in fp32 (casting the live model would round its rotary frequencies to fp16)
    return path, tr.Qwen3ForCausalLM.from_pretrained(path, dtype=torch.float32).eval()


def test_layout_and_logits(checkpoint):
    from Model.Qwen06B_architecture import load_weights
    path, hf = checkpoint
    w, tok = load_weights(path, verbose=False, max_seq_len=MAX_LEN, device="cpu")
    assert len(w["layer_weights"]) == 11 * LAYERS
    for li in range(LAYERS):
        got = [tuple(t.shape) for t in w["layer_weights"][li * 11:(li + 1) * 11]]
        assert got == [s for _, s in S.LAYER_FIELDS]
    assert all(t.dtype == torch.float16 and t.is_contiguous() for t in w["layer_weights"])
    assert w["lm_head_weight"] is w["embed_weight"] and tuple(w["embed_weight"].shape) == (VOCAB, 1024)
    assert tuple(w["cos_table"].shape) == (MAX_LEN, 128) and w["cos_table"].dtype == torch.float16
    assert tok.encode("3 17 250") == [3, 17, 250]
    # every tensor is the checkpoint's tensor of that name
    sd = hf.state_dict()
    names = ("input_layernorm", "self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.q_norm",
             "self_attn.k_norm", "self_attn.o_proj", "post_attention_layernorm", "mlp.gate_proj", "mlp.up_proj",
             "mlp.down_proj")
    for li in range(LAYERS):
        for j, n in enumerate(names):
            assert torch.equal(w["layer_weights"][li * 11 + j].float(), sd[f"model.layers.{li}.{n}.weight"]), (li, n)
    # a decoder on the loaded dictionary computes what transformers computes
    ids = S.make_prompt(9, seed=5, vocab_size=VOCAB)
    with torch.no_grad():
        want = hf(torch.tensor([ids])).logits[0, -1]
    d = OracleDecoder(w, max_seq_len=MAX_LEN, kv_dtype=torch.float32)
    d.prefill(ids[:-1])
    d.step(ids[-1])
    assert (want - d.last_logits).abs().max() < 5e-5


@pytest.mark.gpu
def test_decoder_from_checkpoint_path(checkpoint, built_library):
    """The reference's entry point ``Decoder(model_name=...)`` end to end: checkpoint -> GPU tensors -> greedy tokens
    equal to the oracle's on the same dictionary."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from Model.Qwen06B_architecture import Decoder, load_weights
    path, _ = checkpoint
    eng = Decoder(model_name=path, verbose=False, max_seq_len=MAX_LEN)
    w, _ = load_weights(path, verbose=False, max_seq_len=MAX_LEN, device="cpu")
    text, n_in, n_out = eng.generate("3 17 250 9", 8)
    ids = [3, 17, 250, 9]
    want = OracleDecoder(w, max_seq_len=MAX_LEN).generate_ids(ids, 8)
    want = want[0] if isinstance(want, tuple) else want
    assert n_in == 4 and [int(t) for t in text.split()] == want[:n_out]
