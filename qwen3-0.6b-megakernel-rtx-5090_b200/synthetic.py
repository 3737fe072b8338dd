"""Frozen synthetic model and prompt generators for the Qwen3-0.6B decode path.

No Qwen3 checkpoint or tokenizer is available offline, so every parity test and
benchmark runs on a seeded random-init model of the exact Qwen3-0.6B shape.  The
weight dict produced here has the layout the reference builds in
``Model/Qwen06B_architecture.py:134-159`` (``embed_weight``, flat
``layer_weights`` list of 11 tensors per layer in struct order, tied
``lm_head_weight``, ``final_norm_weight``, fp16 ``cos_table``/``sin_table`` as in
``Model/Qwen06B_architecture.py:126-132``).

Draw order is part of the contract (changing it changes every golden vector):
one ``torch.Generator('cpu')`` seeded with ``seed``; the embedding first, then for
each layer the 11 fields in struct order, then the final norm.  Matrices are
``randn * init_std`` in fp32 rounded to fp16.  Norm weights are exactly 1.0 unless
``norm_std > 0`` (then ``1 + norm_std * randn``, drawn in the same order), which
tests use to make a wrong norm-weight pointer visible.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

HIDDEN_SIZE = 1024
INTERMEDIATE_SIZE = 3072
NUM_Q_HEADS = 16
NUM_KV_HEADS = 8
HEAD_DIM = 128
Q_SIZE = NUM_Q_HEADS * HEAD_DIM
KV_SIZE = NUM_KV_HEADS * HEAD_DIM
NUM_LAYERS = 28
VOCAB_SIZE = 151936
ROPE_THETA = 1_000_000.0
RMS_EPS = 1e-6

# (name, shape builder) in the order of the reference's LDGLayerWeight struct
# (Tools/megakernel/megakernel_5090.cu:91-104).
LAYER_FIELDS = (
    ("input_layernorm", (HIDDEN_SIZE,)),
    ("q_proj", (Q_SIZE, HIDDEN_SIZE)),
    ("k_proj", (KV_SIZE, HIDDEN_SIZE)),
    ("v_proj", (KV_SIZE, HIDDEN_SIZE)),
    ("q_norm", (HEAD_DIM,)),
    ("k_norm", (HEAD_DIM,)),
    ("o_proj", (HIDDEN_SIZE, Q_SIZE)),
    ("post_attention_layernorm", (HIDDEN_SIZE,)),
    ("gate_proj", (INTERMEDIATE_SIZE, HIDDEN_SIZE)),
    ("up_proj", (INTERMEDIATE_SIZE, HIDDEN_SIZE)),
    ("down_proj", (HIDDEN_SIZE, INTERMEDIATE_SIZE)),
)
FIELDS_PER_LAYER = len(LAYER_FIELDS)


@dataclass(frozen=True)
class ModelShape:
    num_layers: int = NUM_LAYERS
    vocab_size: int = VOCAB_SIZE
    max_seq_len: int = 2048


def rope_tables(max_seq_len: int, dtype=torch.float16, theta: float = ROPE_THETA):
    """cos/sin tables ``[max_seq_len, 128]`` with the two halves duplicated."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, HEAD_DIM, 2, dtype=torch.float32) / HEAD_DIM))
    ang = torch.outer(torch.arange(max_seq_len, dtype=torch.float32), inv_freq)
    return (torch.cos(ang).repeat(1, 2).to(dtype).contiguous(),
            torch.sin(ang).repeat(1, 2).to(dtype).contiguous())


def make_weights(seed: int = 0, num_layers: int = NUM_LAYERS, vocab_size: int = VOCAB_SIZE,
                 max_seq_len: int = 2048, init_std: float = 0.02, norm_std: float = 0.0,
                 device: str = "cpu") -> dict:
    """Seeded fp16 weight dict in the reference layout (see module docstring)."""
    gen = torch.Generator("cpu")
    gen.manual_seed(seed)

    def matrix(shape):
        return (torch.randn(shape, generator=gen, dtype=torch.float32) * init_std).to(torch.float16)

    def norm(shape):
        if norm_std > 0.0:
            return (1.0 + norm_std * torch.randn(shape, generator=gen, dtype=torch.float32)).to(torch.float16)
        return torch.ones(shape, dtype=torch.float16)

    embed = matrix((vocab_size, HIDDEN_SIZE))
    layer_weights = []
    for _ in range(num_layers):
        for _, shape in LAYER_FIELDS:
            layer_weights.append(norm(shape) if len(shape) == 1 else matrix(shape))
    final_norm = norm((HIDDEN_SIZE,))
    cos, sin = rope_tables(max_seq_len)

    def put(t):
        return t.to(device).contiguous()

    embed = put(embed)
    return dict(
        embed_weight=embed,
        layer_weights=[put(t) for t in layer_weights],
        final_norm_weight=put(final_norm),
        lm_head_weight=embed,  # tied
        cos_table=put(cos),
        sin_table=put(sin),
    )


def weights_to(weights: dict, device: str) -> dict:
    """Copy of a weight dict on another device, keeping the embedding tie."""
    embed = weights["embed_weight"].to(device).contiguous()
    return dict(
        embed_weight=embed,
        layer_weights=[t.to(device).contiguous() for t in weights["layer_weights"]],
        final_norm_weight=weights["final_norm_weight"].to(device).contiguous(),
        lm_head_weight=embed,
        cos_table=weights["cos_table"].to(device).contiguous(),
        sin_table=weights["sin_table"].to(device).contiguous(),
    )


def make_prompt(n_tokens: int, seed: int = 0, vocab_size: int = VOCAB_SIZE) -> list:
    """``n_tokens`` token IDs uniform in ``[0, vocab_size)`` from their own generator."""
    gen = torch.Generator("cpu")
    gen.manual_seed(seed)
    return torch.randint(0, vocab_size, (n_tokens,), generator=gen, dtype=torch.int64).tolist()


class StubTokenizer:
    """Whitespace-separated decimal token IDs; stands in for the Qwen tokenizer.

    ``encode("17 4 99") == [17, 4, 99]`` and ``decode`` is its inverse, so the
    string-in/string-out ``Decoder.generate`` API and the chat server can be
    exercised without the real vocabulary.
    """

    def __init__(self, eos_token_id: int = -1, vocab_size: int = VOCAB_SIZE):
        self.eos_token_id = eos_token_id
        self.vocab_size = vocab_size

    def encode(self, text, add_special_tokens=False):
        # anything that is not a decimal number (chat-template markup, think tags) is dropped
        return [int(t) % self.vocab_size for t in text.split() if t.isdigit()]

    def decode(self, ids, skip_special_tokens=True):
        return " ".join(str(int(i)) for i in ids)

    def apply_chat_template(self, messages, tokenize=False, add_generation_prompt=True):
        # Content is expected to be decimal IDs already; roles are dropped.
        return " ".join(m["content"] for m in messages)


def weight_bytes_fp16(num_layers: int = NUM_LAYERS, vocab_size: int = VOCAB_SIZE) -> int:
    """Bytes of fp16 weights one decode step must read (LM head once, one embedding row)."""
    per_layer = sum(math.prod(s) for _, s in LAYER_FIELDS) * 2
    return num_layers * per_layer + vocab_size * HIDDEN_SIZE * 2 + HIDDEN_SIZE * 2 + HIDDEN_SIZE * 2


KV_BYTES_PER_POSITION = 2 * NUM_KV_HEADS * HEAD_DIM * 2  # K and V, fp16, one layer


def decode_step_bytes(cache_len: int, num_layers: int = NUM_LAYERS, vocab_size: int = VOCAB_SIZE) -> int:
    """Algorithmic HBM bytes of one batch-1 fp16 decode step attending ``cache_len`` positions.

    weights + KV read over ``cache_len`` positions + one KV row written, all layers.
    """
    return (weight_bytes_fp16(num_layers, vocab_size)
            + num_layers * KV_BYTES_PER_POSITION * cache_len
            + num_layers * KV_BYTES_PER_POSITION)
