"""Small DP CNN on the CPU: samples/s and epsilon after one epoch.

    python -m opacus_b200.benchmarks.cnn_cpu [--impl ours|reference] [--steps N]

60000 synthetic 1x28x28 images (N(0,1) pixels, uniform labels), Poisson sampling
rate 256/60000, SGD lr 0.1, noise multiplier 1.0, clipping norm 1.0, hooks mode,
RDP accountant at delta 1e-5, seed 0.  ``--steps`` limits the number of batches
(the epsilon reported is then that of the steps taken).
"""
import argparse
import json
import os
import sys
import time

import torch
import torch.nn as nn
from torch.utils.data import DataLoader, TensorDataset


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--steps", type=int, default=0, help="0 = one full epoch (234 steps)")
    ap.add_argument("--threads", type=int, default=0)
    args = ap.parse_args()
    import warnings

    warnings.simplefilter("ignore")
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    sys.path.insert(0, root)
    if args.impl == "reference":
        sys.path.insert(0, os.path.join(root, "baseline", "_ref"))
        from opacus import PrivacyEngine
    else:
        from opacus_b200 import PrivacyEngine
    from opacus_b200.models import SmallCNN

    if args.threads:
        torch.set_num_threads(args.threads)
    torch.manual_seed(0)
    n = 60000
    ds = TensorDataset(torch.randn(n, 1, 28, 28), torch.randint(0, 10, (n,)))
    model = SmallCNN()
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    pe = PrivacyEngine(accountant="rdp")
    # batch_size 256 -> len(loader) = 235, sample rate 1/235 ~ 256/60000
    extra = {"skip_param_grads": True} if args.impl == "ours" else {}   # autograd skips the non-private weight gradients
    model, opt, dl = pe.make_private(module=model, optimizer=opt, data_loader=DataLoader(ds, batch_size=256),
                                     noise_multiplier=1.0, max_grad_norm=1.0, **extra)
    crit = nn.CrossEntropyLoss()
    seen, steps, t0 = 0, 0, time.perf_counter()
    for x, y in dl:
        opt.zero_grad()
        if len(x):
            crit(model(x), y).backward()
        opt.step() if len(x) else None
        seen += len(x)
        steps += 1
        if args.steps and steps >= args.steps:
            break
    dt = time.perf_counter() - t0
    print(json.dumps({"impl": args.impl, "metric": "dp_cnn_cpu_samples_per_s", "value": seen / dt, "steps": steps,
                      "samples": seen, "seconds": dt, "epsilon_delta_1e-5": pe.get_epsilon(1e-5),
                      "threads": torch.get_num_threads()}))


if __name__ == "__main__":
    main()
