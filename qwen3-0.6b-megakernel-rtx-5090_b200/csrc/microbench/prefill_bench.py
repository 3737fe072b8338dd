"""Times the tensor-core chunked prefill on the full-size synthetic model and prints prompt tok/s.

    python prefill_bench.py [prompt_tokens=512] [repeats=3] [layers=28]

Also the command profiled for the summaries of the prefill kernels under profiles/ (one chunk of 512
tokens keeps an ncu capture small)."""
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, PKG)

import torch  # noqa: E402

import build  # noqa: E402
import synthetic as S  # noqa: E402


def main():
    n = int(sys.argv[1]) if len(sys.argv) > 1 else 512
    reps = int(sys.argv[2]) if len(sys.argv) > 2 else 3
    layers = int(sys.argv[3]) if len(sys.argv) > 3 else 28
    build.build()
    from Model.Qwen06B_architecture import Decoder
    w = S.weights_to(S.make_weights(seed=0, num_layers=layers, max_seq_len=16), "cuda")
    eng = Decoder(weights=w, tokenizer=S.StubTokenizer(-1), verbose=False, max_seq_len=max(n, 128),
                  prefill_mode="tensor")
    ids = S.make_prompt(n, seed=1)
    eng.prefill_ids(ids)                       # warm-up: workspace, tensor maps
    best = None
    for _ in range(reps):
        eng.reset()
        torch.cuda.synchronize()
        t = time.perf_counter()
        eng.prefill_ids(ids)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t
        best = dt if best is None else min(best, dt)
    flops = 2.0 * n * (layers * 15_728_640 - 6_291_456 - 3_145_728 - 2_097_152)   # last layer: q, k, v only
    print(f"prefill {n} tokens, {layers} layers: {best * 1e3:.2f} ms, {n / best:.0f} prompt tok/s, "
          f"{flops / best / 1e12:.1f} TFLOP/s over the GEMMs' flops")


if __name__ == "__main__":
    main()
