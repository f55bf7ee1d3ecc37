"""Regenerates tests/golden/oracle_vectors.npz from the CPU oracle.

    python tests/golden/make_oracle_vectors.py

The reference has no implementation of the LLM path, so these vectors pin the oracle against
itself over time (a change of the generator, the E4M3/bf16 codecs or the forward pass shows up
as a diff); they are not reference outputs.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402

TINY_QWEN = dict(arch=1, n_layers=2, d_model=256, n_q_heads=4, n_kv_heads=2, head_dim=128, d_ff=512, vocab=1024,
                 max_pos=128, tied=0, eps=1e-6, rope_theta=1e6)
TINY_GPT2 = dict(arch=0, n_layers=2, d_model=128, n_q_heads=2, n_kv_heads=2, head_dim=64, d_ff=512, vocab=512,
                 max_pos=64, tied=1, eps=1e-5, rope_theta=0.0)


def run(cfg, seed, B, S, steps):
    m = O.Model(cfg, seed)
    st = m.new_state(B, S + steps)
    toks = O.gen_tokens(seed + 100, 1, B * S, cfg["vocab"]).reshape(B, S)
    logits = st.prefill(toks, np.full(B, S, np.int32))
    ids = [O.argmax(logits)]
    for _ in range(steps):
        logits = st.decode(ids[-1])
        ids.append(O.argmax(logits))
    st.close()
    m.close()
    return toks, np.stack(ids), logits


def main():
    out = {}
    out["normal_seed7_t3"] = O.gen_normal(7, 3, 64)
    out["tokens_seed1_t1"] = O.gen_tokens(1, 1, 32, 50257)
    q, s = O.gen_qlinear(2, 17, 4, 128)
    out["qlinear_q"], out["qlinear_s"] = q, s
    out["e4m3_table"] = O.e4m3_to_f32(np.arange(256, dtype=np.uint8))
    toks, ids, logits = run(TINY_QWEN, 4, 2, 8, 4)
    out["qwen_tokens"], out["qwen_ids"], out["qwen_last_logits"] = toks, ids, logits
    toks, ids, logits = run(TINY_GPT2, 0, 1, 8, 4)
    out["gpt2_tokens"], out["gpt2_ids"], out["gpt2_last_logits"] = toks, ids, logits
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "oracle_vectors.npz"), **out)
    print({k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
