"""The sharded DP step kernel alone (reduce-scatter + noise + AdamW + all-gather in one launch) on a synthetic
flat space, for every path it has: plain peer loads / stores or the NVLink multicast address, whole grid or the
capped grid a piece uses beside the weight-gradient GEMMs.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m opacus_b200.benchmarks.sharded_step [--params 1235814400] [--iters 10] [--json out.json]

Times are CUDA-event medians, max over ranks; the flat buffers (several GB) exceed the L2.  The roofline time is the
larger of the HBM bytes of a rank (fp32 gradient read, master / two moments read + written, parameters written) over
the measured copy bandwidth and the NVLink bytes leaving a GPU (its gradient read by the other owners, its new
weights published) over 770 GB/s, the measured peer-copy bandwidth per direction.
"""
import argparse
import datetime
import json
import os

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import _cuda
from ..parallel.sharded import ShardedDataParallel
from .kernels import _peaks

LINK_GBS = 770.0


class _Flat(nn.Module):
    def __init__(self, n):
        super().__init__()
        self.w = nn.Parameter(torch.zeros(n, device="cuda"))

    def forward(self, x):
        return x


class _Opt:
    """The part of a DP optimizer the engine's step reads."""

    def __init__(self, inner):
        self.original_optimizer = inner
        self.loss_reduction = "mean"
        self.step_hook = None
        self.generator = None
        self.secure_mode = False
        self._is_last_step_skipped = False

    def _check_skip_next_step(self):
        return False

    def _grad_denominator(self):
        return 8.0

    def _noise_std(self):
        return 0.8


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--params", type=int, default=1235814400, help="elements of the flat space (Llama-3.2-1B, tied)")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--blocks", type=int, nargs="*", default=[0, 148], help="grid caps to time (0: whole grid)")
    ap.add_argument("--json", default=None)
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29583")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    rank, world = dist.get_rank(), dist.get_world_size()
    _, hbm_gbs, src = _peaks()
    rows = []
    # (multicast address used for the reduce, for the publish)
    variants = ((False, False), (False, True), (True, True)) if world > 1 else ((False, False),)
    model = _Flat(args.params)
    eng = ShardedDataParallel(model, process_group=None, step_pieces=1)
    have_mc = eng.multicast
    opt = _Opt(torch.optim.AdamW(model.parameters(), lr=1e-4))
    eng.flat_grad().normal_()
    for mc_reduce, mc_publish in variants:
        if (mc_reduce or mc_publish) and not have_mc:
            if rank == 0:
                print("no NVLink multicast address on this fabric: multimem paths not measured")
            break
        eng.multicast = mc_reduce or mc_publish
        eng.multicast_reduce, eng.multicast_publish = mc_reduce, mc_publish
        for cap in args.blocks:
            eng.single_launch_blocks = cap

            def one():
                for p in eng._params:
                    p._dp_grad_fresh = False
                eng._optimizer_step(opt)

            for _ in range(3):
                one()
            torch.cuda.synchronize()
            ts = []
            for _ in range(args.iters):
                dist.barrier()
                torch.cuda.synchronize()
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                one()
                e.record()
                torch.cuda.synchronize()
                ts.append(s.elapsed_time(e))
            _cuda.check_status()
            ts.sort()
            t = torch.tensor([ts[len(ts) // 2]], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t)
            own = eng.slice_len
            # gradient reads this GPU's memory serves (its whole buffer) + master / two moments read and written for
            # the owned share + the parameters written into this GPU's compute buffer
            hbm = eng.total * 4 + own * 4 * 6 + eng.total * 2
            link = (eng.total * 4 * (world - 1) // world + own * 2 * (1 if mc_publish else world - 1)) if world > 1 else 0
            roof = max(hbm / (hbm_gbs * 1e6), link / (LINK_GBS * 1e6))
            rows.append(dict(world=world, multicast_reduce=mc_reduce, multicast_publish=mc_publish, max_blocks=cap, ms=ms,
                             hbm_bytes=int(hbm),
                             nvlink_bytes_out=int(link), roofline_ms=roof, frac_of_roofline=roof / ms))
            if rank == 0:
                print(f"world {world} multimem reduce {int(mc_reduce)} publish {int(mc_publish)} blocks {cap or 'all':>4}: {ms:7.3f} ms   "
                      f"HBM {hbm / 1e9:5.2f} GB  NVLink out {link / 1e9:5.2f} GB  roofline {roof:6.3f} ms "
                      f"({roof / ms:.2f} of {src})", flush=True)
    if rank == 0 and args.json:
        with open(args.json, "w") as f:
            json.dump(rows, f, indent=1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
