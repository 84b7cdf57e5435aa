"""Headline benchmark: DP-SGD tokens/s on a Llama-3.2-1B-shaped decoder with
ghost clipping and DP-AdamW (seq 1024, per-GPU batch 8, C = 1.0, sigma = 0.8),
on N GPUs of one node.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the unmodified reference library, same model and config

Prints one JSON line (rank 0).  ``value`` is device-timed (CUDA events, max over
ranks) with the step's inputs already on the GPU; ``e2e`` repeats the
measurement through the public API with a pinned-host -> device copy of every
step's batch and a device -> host read of its loss inside the timed region.
Data are synthetic token ids, weights are randomly initialised.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading

import torch
import torch.distributed as dist
import torch.nn as nn

REPO = os.path.dirname(os.path.abspath(__file__))
SEQ = 1024
PER_GPU_BATCH = 8
SIGMA = 0.8
CLIP = 1.0
LR = 1e-4
DATASET_BATCHES = 64          # synthetic dataset size = this many global batches


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--engine", default="sharded", choices=["sharded", "plain"],
                    help="ours: sharded data-parallel engine (default) or, on one GPU, the plain ghost path")
    ap.add_argument("--ce", default="fused", choices=["fused", "torch"],
                    help="ours: FusedCrossEntropyLoss on bf16 logits, or nn.CrossEntropyLoss on logits.float()")
    ap.add_argument("--untied", action="store_true",
                    help="ours: control run with untied embeddings (the reference arm's parameter set); not the default")
    ap.add_argument("--plain-model", action="store_true",
                    help="ours: control run on the stock-PyTorch model definition the reference arm uses (no fused "
                         "cross entropy / RoPE / SwiGLU / add+RMSNorm kernels in the model); not the default")
    ap.add_argument("--layers", type=int, default=None, help="debug only: fewer layers (result is not a benchmark)")
    ap.add_argument("--vocab", type=int, default=None, help="debug only")
    ap.add_argument("--seq", type=int, default=SEQ, help="debug only")
    ap.add_argument("--batch", type=int, default=PER_GPU_BATCH, help="debug only")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        busy = sorted(sm)[len(sm) // 2:] if sm else []
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def setup_dist(n):
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    return rank, local, world


def make_model(args, tie: bool, plain: bool = False):
    """Llama-3.2-1B-shaped model.  ``plain``: the stand-alone stock-PyTorch definition under
    ``baseline/`` (reference arm: nothing of this package on its path); otherwise this package's model."""
    if plain:
        sys.path.insert(0, os.path.join(REPO, "baseline"))
        from llama_plain import Llama, llama_1b_config
    else:
        sys.path.insert(0, REPO)
        from opacus_b200.models import Llama, llama_1b_config

    kw = {}
    if args.layers:
        kw["n_layers"] = args.layers
    if args.vocab:
        kw["vocab_size"] = args.vocab
    cfg = llama_1b_config(tie_embeddings=tie, **kw)
    torch.manual_seed(1234)
    with torch.device("cuda"):
        model = Llama(cfg)
    return model, cfg


def make_data(cfg, args, world, rank):
    """Pinned host batches (ids and next-token labels) for this rank."""
    g = torch.Generator().manual_seed(100 + rank)
    n = 16
    toks = torch.randint(0, cfg.vocab_size, (n, args.batch, args.seq + 1), generator=g)
    ids = toks[:, :, :-1].contiguous().pin_memory()
    labels = toks[:, :, 1:].contiguous().pin_memory()
    return ids, labels


# --------------------------------------------------------------------------- ours
def build_ours(args, rank, world):
    from torch.utils.data import DataLoader, TensorDataset

    from opacus_b200 import PrivacyEngine
    from opacus_b200.distributed import DifferentiallyPrivateDistributedDataParallel as DPDDP

    plain = getattr(args, "plain_model", False)
    model, cfg = make_model(args, tie=not getattr(args, "untied", False), plain=plain)
    module = model
    mode = "ghost"
    if args.engine == "sharded":
        from opacus_b200.utils.fsdp_utils import FSDP2Wrapper

        module = FSDP2Wrapper(model)          # -> ShardedDataParallel: bf16 compute weights, sharded fp32 state
        mode = "ghost_fsdp"
    elif world > 1:
        module = DPDDP(model)
    optimizer = torch.optim.AdamW(model.parameters(), lr=LR)
    n_data = DATASET_BATCHES * args.batch * world
    ds = TensorDataset(torch.zeros(n_data, 1, dtype=torch.long))     # only its length matters (sample rate)
    dl = DataLoader(ds, batch_size=args.batch * world)
    engine = PrivacyEngine(accountant="rdp")
    fused_ce = args.ce == "fused" and not plain
    if fused_ce:
        from opacus_b200.layers import FusedCrossEntropyLoss

        base_criterion = FusedCrossEntropyLoss()      # fp32 loss straight from the bf16 logits, bf16 gradient
    else:
        base_criterion = nn.CrossEntropyLoss()
    module, optimizer, criterion, _ = engine.make_private(
        module=module, optimizer=optimizer, criterion=base_criterion, data_loader=dl,
        noise_multiplier=SIGMA, max_grad_norm=CLIP, grad_sample_mode=mode, poisson_sampling=False)

    def step(ids, labels):
        optimizer.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            logits = module(ids)
        if not fused_ce:
            logits = logits.float()
        loss = criterion(logits.view(-1, logits.shape[-1]), labels.reshape(-1), shape=(ids.shape[0], ids.shape[1]))
        loss.backward()
        optimizer.step()
        return loss.detach()

    step.engine = module._module if args.engine == "sharded" else None
    return step, cfg, engine, mode


# ---------------------------------------------------------------------- reference
def build_reference(args, rank, world):
    ref = os.path.join(REPO, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "opacus")):
        raise RuntimeError("reference not installed under baseline/_ref")
    sys.path.insert(0, ref)
    from opacus import PrivacyEngine
    from torch.utils.data import DataLoader, TensorDataset

    # ghost clipping in the reference rejects shared parameters, so the embedding is untied
    model, cfg = make_model(args, tie=False, plain=True)
    mode = "ghost"
    module = model
    if world > 1:
        from opacus.utils.fsdp_utils import FSDP2Wrapper
        from torch.distributed.fsdp import MixedPrecisionPolicy

        module = FSDP2Wrapper(model, mp_policy=MixedPrecisionPolicy(param_dtype=torch.bfloat16,
                                                                    reduce_dtype=torch.float32))
        mode = "ghost_fsdp"
    optimizer = torch.optim.AdamW(module.parameters(), lr=LR)
    n_data = DATASET_BATCHES * args.batch * world
    ds = TensorDataset(torch.zeros(n_data, 1, dtype=torch.long))
    dl = DataLoader(ds, batch_size=args.batch * world)
    engine = PrivacyEngine(accountant="rdp")
    module, optimizer, criterion, _ = engine.make_private(
        module=module, optimizer=optimizer, criterion=nn.CrossEntropyLoss(), data_loader=dl,
        noise_multiplier=SIGMA, max_grad_norm=CLIP, grad_sample_mode=mode, poisson_sampling=False)
    use_autocast = world == 1

    def step(ids, labels):
        optimizer.zero_grad(set_to_none=True)
        if use_autocast:
            with torch.autocast("cuda", dtype=torch.bfloat16):
                logits = module(ids)
        else:
            logits = module(ids)
        loss = criterion(logits.float().view(-1, logits.shape[-1]), labels.reshape(-1), shape=(ids.shape[0], ids.shape[1]))
        loss.backward()
        optimizer.step()
        return loss.detach()

    return step, cfg, engine, mode


def max_over_ranks(value: float, world: int) -> float:
    if world == 1:
        return value
    t = torch.tensor([value], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier(world):
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def main():
    args = parse()
    if not torch.cuda.is_available():
        print(json.dumps({"impl": args.impl, "unavailable": "no CUDA device visible"}))
        return 0
    rank, local, world = setup_dist(args.gpus)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    need_pg = world > 1 or (args.impl == "ours" and args.engine == "sharded")
    if need_pg and not dist.is_initialized():
        import datetime

        dist.init_process_group("nccl", device_id=torch.device("cuda", local),
                                timeout=datetime.timedelta(seconds=180))

    try:
        if args.impl == "reference":
            step, cfg, engine, mode = build_reference(args, rank, world)
        else:
            step, cfg, engine, mode = build_ours(args, rank, world)
    except Exception as e:  # the reference arm reports, it does not crash the driver
        if args.impl == "reference":
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": f"{type(e).__name__}: {e}"[:300]}))
            return 0
        raise

    ids_h, labels_h = make_data(cfg, args, world, rank)
    nb = ids_h.shape[0]
    ids_d, labels_d = ids_h.cuda(), labels_h.cuda()
    tokens_per_step = args.batch * args.seq * world

    # ---- device-timed: inputs resident on the GPU
    for i in range(args.warmup):
        step(ids_d[i % nb], labels_d[i % nb])
    barrier(world)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier(world)
    start.record()
    for i in range(args.steps):
        step(ids_d[i % nb], labels_d[i % nb])
    end.record()
    barrier(world)
    ms = max_over_ranks(start.elapsed_time(end), world) / args.steps

    # ---- end to end: pinned host -> device copy of each batch, loss read back each step
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    last = 0.0
    e0.record()
    for i in range(args.steps):
        x = ids_h[i % nb].to("cuda", non_blocking=True)
        y = labels_h[i % nb].to("cuda", non_blocking=True)
        last = float(step(x, y).item())
    e1.record()
    barrier(world)
    e2e_ms = max_over_ranks(e0.elapsed_time(e1), world) / args.steps
    clocks = sampler.stop() if rank == 0 else None
    # epsilon of exactly warmup + 2 * steps accounted steps, the same count in both arms
    eps = None
    try:
        eps = float(engine.get_epsilon(1e-5))
    except Exception:
        pass
    sharded = getattr(step, "engine", None)
    replicas = replicas_identical(sharded, world) if sharded is not None else None
    nvlink = nvlink_bytes_per_step(sharded) if sharded is not None else None
    # every rank runs the profiled extra step (it contains collectives / peer barriers)
    per_step = count_launches(step, ids_d[0], labels_d[0]) if args.impl == "ours" else None

    if rank == 0:
        launches = None if per_step is None else per_step * args.steps
        full = args.layers is None and args.vocab is None and args.seq == SEQ and args.batch == PER_GPU_BATCH
        out = {
            "metric": "dp_sgd_tokens_per_s_llama1b_ghost_clip",
            "impl": args.impl,
            "value": tokens_per_step / (ms / 1e3),
            "unit": "tokens/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": ms,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "bf16",
            "data": "synthetic token ids (uniform over vocab), random-init weights",
            "config": {
                "model": "llama-3.2-1b-shaped" if full else "DEBUG-reduced",
                "layers": cfg.n_layers, "d_model": cfg.d_model, "vocab": cfg.vocab_size,
                "tied_embeddings": cfg.tie_embeddings,
                "model_definition": "stock PyTorch (baseline/llama_plain.py)" if (args.impl == "reference" or
                                                                                  getattr(args, "plain_model", False))
                else "opacus_b200.models.Llama (fused RoPE / SwiGLU / add+RMSNorm / cross entropy)",
                "global_batch": args.batch * world, "seq_len": args.seq,
                "parallelism": ("single" if world == 1 else f"dp{world}") + f" ({mode})",
                "optimizer": "DP-AdamW lr 1e-4", "noise_multiplier": SIGMA, "max_grad_norm": CLIP,
                "l2_policy": "inputs and activations per step (several GB) exceed the 126 MB L2; no explicit flush",
                "epsilon_at_delta_1e-5_after_run": eps,
            },
            "clocks": clocks,
            "e2e": {"value": tokens_per_step / (e2e_ms / 1e3), "unit": "tokens/s",
                    "h2d_bytes_per_step": int(2 * args.batch * args.seq * 8), "d2h_bytes_per_step": 4,
                    "ms_per_step": e2e_ms, "last_loss": last},
            "gpu_launches": launches,
        }
        if replicas is not None:
            out["replicas_identical"] = replicas
        if nvlink is not None:
            out["nvlink_bytes_per_step"] = nvlink
            out["step_path"] = {"multicast": bool(sharded.multicast), "pieces": sharded.pieces,
                                "launches_last_step": sharded.last_step_launches}
        print(json.dumps(out))
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    return 0


def replicas_identical(engine, world):
    """After the timed region: do all ranks hold the same compute weights, bit for bit?  (Two 64-bit
    checksums of the flat parameter buffer, compared across ranks.)"""
    flat = engine.flat_param()
    words = flat.view(torch.int16 if flat.element_size() == 2 else torch.int32).to(torch.int64)
    weights = torch.arange(words.numel(), device=words.device, dtype=torch.int64) % 65521 + 1
    sums = torch.stack([words.sum(), (words * weights).sum()])
    if world == 1:
        return True
    all_sums = [torch.empty_like(sums) for _ in range(world)]
    dist.all_gather(all_sums, sums)
    return all(bool(torch.equal(all_sums[0], t)) for t in all_sums[1:])


def nvlink_bytes_per_step(engine):
    """Bytes that leave one GPU over NVLink in the step kernel: its fp32 gradient sums read by the other owners,
    and the new weights of its stripes (one copy into the switch with multicast stores, world - 1 copies without)."""
    w = engine.world
    if w == 1:
        return 0
    reduce_out = engine.total * 4 * (w - 1) // w
    publish_out = engine.slice_len * engine.flat_param().element_size() * (1 if engine.multicast else w - 1)
    return int(reduce_out + publish_out)


def count_launches(step, ids, labels):
    """Number of launches of this package's own kernels in one step (kernel names in the dpk namespace)."""
    try:
        from torch.profiler import ProfilerActivity, profile

        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            step(ids, labels)
            torch.cuda.synchronize()
        return int(sum(e.count for e in prof.key_averages() if "dpk" in e.key))
    except Exception:
        return None


if __name__ == "__main__":
    sys.exit(main())
