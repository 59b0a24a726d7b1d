"""LM1B training without distribution: a plain PyTorch loop over the same model and synthetic Zipf ids.

It is the single-process reference that ``lm1b_train.py`` is compared against (reference:
``examples/lm1b/lm1b_train_eager.py``): same model, optimizer, gradient scaling and clipping, no AutoDist object.
"""
import argparse
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from autodist_b200.models.lm1b import LM1B, LM1BConfig, zipf_tokens  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch_size", type=int, default=128)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--tiny", action="store_true")
    args = ap.parse_args()
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    cfg = LM1BConfig.tiny() if args.tiny else LM1BConfig()
    model = LM1B(cfg).to(dev)
    sparse, dense = model.sparse_grad_parameters(), model.dense_parameters()
    opt = torch.optim.Adagrad(model.parameters(), lr=0.2, initial_accumulator_value=1.0)
    data = {k: v.to(dev) for k, v in zipf_tokens(args.batch_size, cfg.num_steps, cfg.vocab_size).items()}
    t0 = time.time()
    for step in range(1, args.steps + 1):
        opt.zero_grad(set_to_none=True)
        loss = model(data["x"], data["y"])
        loss.backward()
        torch.nn.utils.clip_grad_norm_(dense, cfg.max_grad_norm)
        opt.step()
        if step % 10 == 0:
            if dev.type == "cuda":
                torch.cuda.synchronize()
            wps = 10 * args.batch_size * cfg.num_steps / (time.time() - t0)
            print(f"step {step} loss {float(loss):.3f} {wps:.0f} words/s ({len(sparse)} row-sparse tables)", flush=True)
            t0 = time.time()


if __name__ == "__main__":
    main()
