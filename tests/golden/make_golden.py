"""Writes the small golden fixtures of this directory from the oracle.

    python tests/golden/make_golden.py

synth_golden.json  -- bit patterns of the counter-based generator (seed, tensor id, index)
small_llama_golden.npz -- greedy tokens and first-step logits of BASELINE config 1 (4 layers,
    hidden 256, 8 heads, MLP 688, vocab 1024; 32-token prompt, 64 steps) from the oracle, so the
    GPU parity test also has a committed reference that does not depend on re-running the oracle.

Both files are written by this repository's own oracle: they are regression fixtures (they catch a change of
the oracle or of the generator), not vectors of the reference, which cannot run here.
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", "..", "oracle"))
import luminal_oracle as O  # noqa: E402


def main():
    seed, tid, n, sigma = 1234, 17, 16, 0.02
    vals = O.synth_normal(seed, tid, (n,), sigma)
    json.dump({"seed": seed, "tensor_id": tid, "n": n, "sigma": sigma,
               "bits": vals.view(np.uint32).tolist(),
               "tokens": O.synth_tokens(seed, tid, (8,), 1024).tolist()},
              open(os.path.join(HERE, "synth_golden.json"), "w"))
    cfg = O.CONFIGS["small_llama"]
    w = O.synth_llama_weights(cfg, seed=1234)
    prompt = O.synth_tokens(1234, 1000, (1, 32), cfg["vocab"])
    tok, log = O.CachedLlama(w, cfg, 1, 128).greedy(prompt, 64)
    np.savez_compressed(os.path.join(HERE, "small_llama_golden.npz"), prompt=prompt, tokens=tok,
                        logits_first=log[:, 0], logits_last=log[:, -1])


if __name__ == "__main__":
    main()
