"""Generates tests/golden/*.npz from the CPU oracle.

Two kinds of fixture:
  closed_forms.npz   the constant-weight known answers of the reference's DeviceBackend test
                     (tests/mixed_linear_parity.cu:204-281): Q8_0 scale 0.5, every quant 1,
                     input x -> y = cols * 0.5 * x.
  tiny_streams.npz   the oracle's own outputs on the tiny qwen35 configuration (seeded weights,
                     seeded prompt): greedy token stream, MTP k=1 stream, first-step logits.  These pin
                     the oracle against drift; the GPU tests compare against the live oracle as well.
Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    O = entry.load_oracle()
    pkg = entry.load_package()
    # closed forms
    rows, cols = 128, 512
    blocks = np.zeros(rows * (cols // 32) * 34, np.uint8).reshape(-1, 34)
    blocks[:, 0:2] = np.frombuffer(np.float16(0.5).tobytes(), np.uint8)
    blocks[:, 2:] = 1
    batch = 64
    x = np.repeat(((np.arange(batch) + 1) / 64.0).astype(np.float32)[:, None], cols, 1)
    y = O.matmul_engine(blocks.reshape(-1), rows, cols, x)
    np.savez(os.path.join(HERE, "closed_forms.npz"), rows=rows, cols=cols, x_first_col=x[:, 0],
             expected=(cols * 0.5 * x[:, 0]).astype(np.float32), oracle_y_col0=y[:, 0])
    # tiny streams
    cfg = pkg.configs.tiny()
    ocfg = O.ModelConfig(**cfg.as_dict())
    m = O.Model(ocfg, pkg.configs.MODEL_SEED)
    prompt = O.synth_prompt(pkg.configs.PROMPT_SEED + 1, cfg.vocab_size, 64)
    s = O.Seq(m, 256)
    s.prefill(prompt, 64)
    logits0 = s.last_logits(1)[0].copy()
    greedy = [s.cur_token]
    while len(greedy) < 32:
        greedy.append(s.greedy_step())
    s2 = O.Seq(m, 256)
    s2.prefill(prompt, 64)
    mtp = [s2.cur_token]
    while len(mtp) < 32:
        toks, _, _ = s2.mtp_step(1)
        mtp += toks
    np.savez(os.path.join(HERE, "tiny_streams.npz"), prompt=prompt, greedy=np.array(greedy, np.int32),
             mtp_k1=np.array(mtp[:32], np.int32), logits0_top=np.sort(logits0)[-8:], logits0_argmax=int(np.argmax(logits0)),
             logits0_sample=logits0[::64])
    print("wrote fixtures")


if __name__ == "__main__":
    main()
