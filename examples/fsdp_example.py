"""Sequence classification with ghost clipping on sharded data parallelism, with a checkpoint and a resume.

    python examples/fsdp_example.py                                  # one GPU
    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 examples/fsdp_example.py

A small Transformer encoder classifies synthetic token sequences (class 1 draws most of its tokens from the upper half
of the vocabulary, class 0 from the lower half, so the loss really falls).  ``FSDP2Wrapper`` hands the model to this package's sharded engine: bf16 compute weights, fp32 master weights
and AdamW moments sharded over the ranks, gradients reduced and parameters published inside the step kernel.  Two
parameter groups (weight decay on matrices, none on norms and biases) show that groups may differ in learning rate
and weight decay.  Half way through, the run saves a checkpoint with ``PrivacyEngine.save_checkpoint`` (model in fp32
master precision, optimiser state in ``torch.optim`` layout, accountant history), builds everything again from
scratch, loads the file and continues; the privacy budget carries on from where it was.

Counterpart in the reference: ``examples/fsdp_example.py``.
"""
import argparse
import os
import sys
import tempfile

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.utils.data import DataLoader, TensorDataset

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))   # run from a source checkout

from opacus_b200 import PrivacyEngine  # noqa: E402
from opacus_b200.layers import DPMultiheadAttention  # noqa: E402
from opacus_b200.utils.fsdp_utils import FSDP2Wrapper  # noqa: E402


class Block(nn.Module):
    def __init__(self, d, heads):
        super().__init__()
        self.norm1, self.norm2 = nn.LayerNorm(d), nn.LayerNorm(d)
        self.attn = DPMultiheadAttention(d, heads, batch_first=True)
        self.up, self.down = nn.Linear(d, 4 * d), nn.Linear(4 * d, d)

    def forward(self, x):
        h = self.norm1(x)
        x = x + self.attn(h, h, h, need_weights=False)[0]
        return x + self.down(torch.nn.functional.gelu(self.up(self.norm2(x))))


class Classifier(nn.Module):
    def __init__(self, vocab, d, heads, layers, seq, classes):
        super().__init__()
        self.tok = nn.Embedding(vocab, d)
        self.pos = nn.Embedding(seq, d)
        self.blocks = nn.ModuleList([Block(d, heads) for _ in range(layers)])
        self.norm = nn.LayerNorm(d)
        self.head = nn.Linear(d, classes)

    def forward(self, ids):
        x = self.tok(ids) + self.pos(torch.arange(ids.shape[1], device=ids.device).expand_as(ids))
        for blk in self.blocks:
            x = blk(x)
        return self.head(self.norm(x).mean(dim=1))


def make_batch(gen, batch, seq, vocab, device):
    labels = torch.randint(0, 2, (batch,), generator=gen)
    upper = torch.rand(batch, seq, generator=gen) < (0.25 + 0.5 * labels[:, None].float())
    ids = torch.randint(0, vocab // 2, (batch, seq), generator=gen) + upper.long() * (vocab // 2)
    return ids.to(device), labels.to(device)


def build(args, world):
    torch.manual_seed(0)
    model = Classifier(args.vocab, args.d_model, 4, args.layers, args.seq, 2).cuda()
    module = FSDP2Wrapper(model)
    decay = [p for p in model.parameters() if p.dim() >= 2]
    plain = [p for p in model.parameters() if p.dim() < 2]
    optimizer = torch.optim.AdamW([{"params": decay, "weight_decay": 0.01},
                                   {"params": plain, "weight_decay": 0.0, "lr": 2 * args.lr}], lr=args.lr)
    loader = DataLoader(TensorDataset(torch.zeros(args.batch * world * 64, 1)), batch_size=args.batch * world)
    engine = PrivacyEngine(accountant="rdp")
    module, optimizer, criterion, _ = engine.make_private(
        module=module, optimizer=optimizer, criterion=nn.CrossEntropyLoss(), data_loader=loader,
        noise_multiplier=args.sigma, max_grad_norm=1.0, grad_sample_mode="ghost_fsdp", poisson_sampling=False)
    return engine, module, optimizer, criterion


def train(module, optimizer, criterion, gen, args, steps, rank, first):
    for step in range(first, first + steps):
        ids, labels = make_batch(gen, args.batch, args.seq, args.vocab, "cuda")
        optimizer.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            logits = module(ids)
        loss = criterion(logits.float(), labels)
        loss.backward()
        optimizer.step()
        if rank == 0 and step % 5 == 0:
            acc = (logits.argmax(dim=1) == labels).float().mean().item()
            print(f"step {step:3d}  loss {loss.item():.3f}  batch accuracy {acc:.2f}", flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--d-model", type=int, default=128)
    ap.add_argument("--vocab", type=int, default=1000)
    ap.add_argument("--seq", type=int, default=64)
    ap.add_argument("--batch", type=int, default=256, help="per GPU")
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--lr", type=float, default=2e-3)
    ap.add_argument("--sigma", type=float, default=0.3)
    ap.add_argument("--checkpoint", default=None, help="where to write the checkpoint (default: a temporary file)")
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    for k, v in (("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", "29546"), ("RANK", "0"), ("WORLD_SIZE", "1")):
        os.environ.setdefault(k, v)
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    gen = torch.Generator().manual_seed(100 + rank)
    half = args.steps // 2

    engine, module, optimizer, criterion = build(args, world)
    train(module, optimizer, criterion, gen, args, half, rank, 0)
    path = args.checkpoint or os.path.join(tempfile.gettempdir(), "opacus_b200_fsdp_example.pt")
    # gathering the sharded state is collective: every rank calls save_checkpoint, rank 0's file is the one kept
    target = path if rank == 0 else os.devnull
    engine.save_checkpoint(path=target, module=module, optimizer=optimizer)
    dist.barrier()
    if rank == 0:
        print(f"checkpoint written after {half} steps, eps = {engine.get_epsilon(1e-5):.2f}; starting over from it")

    engine, module, optimizer, criterion = build(args, world)        # a fresh process would do exactly this
    # map_location: the file holds rank 0's tensors; no rank should open a context on another rank's GPU for them
    engine.load_checkpoint(path=path, module=module, optimizer=optimizer, torch_load_kwargs={"map_location": "cpu"})
    train(module, optimizer, criterion, gen, args, args.steps - half, rank, half)
    if rank == 0:
        print(f"done: {args.steps} steps accounted, eps(1e-5) = {engine.get_epsilon(1e-5):.2f}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
