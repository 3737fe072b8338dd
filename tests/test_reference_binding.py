"""The reference project's own torch binding and Python layer, driving this repository's library.

``tests/reference_binding/build_ref_binding.py`` compiles the reference's ``Tools/megakernel/qwen_ops.cpp`` unmodified
against ``libqwen_megakernel.so`` and stages the reference's ``Model/Qwen06B_architecture.py`` under the git-ignored
``baseline/_ref/``.  The tests here run them in a child process (their module names are the same as this
repository's own ``qwen_megakernel_C`` / ``Model``) and are skipped when that build has not been made.
"""

import glob
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
PKG = os.path.join(ROOT, "qwen3-0.6b-megakernel-rtx-5090_b200")
GOLDEN = os.path.join(ROOT, "tests", "golden", "full_seed0_prompt32.json")


def _staged():
    return bool(glob.glob(os.path.join(REF, "qwen_megakernel_C*.so"))) and \
        os.path.exists(os.path.join(REF, "Model", "Qwen06B_architecture.py"))


needs_ref = pytest.mark.skipif(not _staged(), reason="reference binding not built (tests/reference_binding/build_ref_binding.py)")


def _child(code: str, timeout: int = 600) -> str:
    env = dict(os.environ, PYTHONPATH=REF)
    proc = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=timeout, env=env, cwd=REF)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-4000:]
    return proc.stdout


@needs_ref
def test_reference_binding_loads_and_resolves_the_launchers(built_library):
    """The extension's undefined launch_ldg_* symbols resolve against libqwen_megakernel.so at load time
    (no GPU needed), and it reports the reference's ABI version."""
    out = _child("import torch, qwen_megakernel_C as C\n"
                 "print(C.__file__)\nprint(C.abi_version())\n"
                 "print(all(hasattr(C, n) for n in ('decode', 'generate_nosync', 'prefill')))")
    lines = out.strip().splitlines()
    assert lines[0].startswith(REF) and lines[1] == "2" and lines[2] == "True"


CHILD_GPU = r"""
import json, sys
sys.path.insert(0, {ref!r})
import torch
import Model.Qwen06B_architecture as ARCH          # the reference's file
assert ARCH.__file__.startswith({ref!r})
sys.path.append({pkg!r})                            # only for the seeded weight generator and the stub tokenizer
import synthetic as S
g = json.load(open({golden!r}))
w = S.weights_to(S.make_weights(seed=0, max_seq_len=ARCH.MAX_SEQ_LEN), "cuda")     # fp16 tables for 2048 positions, as the reference builds them
dec = ARCH.Decoder(weights=w, tokenizer=S.StubTokenizer(-1), verbose=False)
text, n_in, n_out = dec.generate(" ".join(map(str, g["prompt"])), max_tokens=32)
toks = [int(t) for t in text.split()]
# token-by-token through the decode op as well
dec.reset()
cur = None
for t in g["prompt"]:
    cur = dec.step(t)
print(json.dumps(dict(tokens=toks, n_in=n_in, n_out=n_out, first_by_step=cur)))
"""


@needs_ref
@pytest.mark.gpu
def test_reference_decoder_on_this_library_matches_the_oracle(built_library):
    """The reference's unmodified Decoder (its 2048-position cache, its scratch tensors, its request logic), bound
    through its unmodified qwen_ops.cpp, produces the oracle's 32 greedy tokens on the seed-0 full model."""
    out = _child(CHILD_GPU.format(ref=REF, pkg=PKG, golden=GOLDEN), timeout=900)
    res = json.loads(out.strip().splitlines()[-1])
    g = json.load(open(GOLDEN))
    assert res["n_in"] == len(g["prompt"]) and res["n_out"] == 32
    assert res["tokens"] == g["tokens"]
    assert res["first_by_step"] == g["tokens"][0]
