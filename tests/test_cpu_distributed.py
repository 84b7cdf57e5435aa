"""Host-side logic of the multi-process paths on CPU (gloo, 2 ranks): data-parallel
DP optimizers against a single-process run, tensor-parallel ghost clipping against
the unsharded model, the distributed Poisson sampler, and failure detection by a
short process-group timeout when a rank never joins a collective."""
import datetime
import os
import socket
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, fn, out_dir, timeout_s):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))
    try:
        result = fn(rank, world)
        torch.save(result, os.path.join(out_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


def _run(fn, world=2, timeout_s=60):
    out_dir = tempfile.mkdtemp()
    mp.spawn(_worker, args=(world, _free_port(), fn, out_dir, timeout_s), nprocs=world, join=True)
    return [torch.load(os.path.join(out_dir, f"r{r}.pt"), weights_only=False) for r in range(world)]


def _mlp():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(12, 16), nn.Tanh(), nn.LayerNorm(16), nn.Linear(16, 4))


def _data():
    g = torch.Generator().manual_seed(1)
    return torch.randn(8, 12, generator=g), torch.randint(0, 4, (8,), generator=g)


class _DDPJob:
    def __init__(self, mode):
        self.mode = mode

    def __call__(self, rank, world):
        mode = self.mode
        from torch.utils.data import DataLoader, TensorDataset

        from opacus_b200 import PrivacyEngine
        from opacus_b200.distributed import DifferentiallyPrivateDistributedDataParallel as DPDDP

        x, y = _data()
        model = DPDDP(_mlp())
        opt = torch.optim.SGD(model.parameters(), lr=0.5)
        dl = DataLoader(TensorDataset(x, y), batch_size=8)
        out = PrivacyEngine(accountant="rdp").make_private(
            module=model, optimizer=opt, data_loader=dl, noise_multiplier=0.0, max_grad_norm=0.2,
            grad_sample_mode=mode, poisson_sampling=False)
        m, o = out[0], out[1]
        crit = out[2] if mode == "ghost" else nn.CrossEntropyLoss()
        xs, ys = x[rank::world], y[rank::world]
        for _ in range(2):
            o.zero_grad()
            crit(m(xs), ys).backward()
            o.step()
        return [p.detach().clone() for p in model.parameters()]


@pytest.mark.parametrize("mode", ["hooks", "ghost"])
def test_ddp_equals_single_process(mode):
    from torch.utils.data import DataLoader, TensorDataset

    from opacus_b200 import PrivacyEngine

    got = _run(_DDPJob(mode))
    x, y = _data()
    model = _mlp()
    opt = torch.optim.SGD(model.parameters(), lr=0.5)
    m, o, _ = PrivacyEngine(accountant="rdp").make_private(
        module=model, optimizer=opt, data_loader=DataLoader(TensorDataset(x, y), batch_size=8),
        noise_multiplier=0.0, max_grad_norm=0.2, poisson_sampling=False)
    for _ in range(2):
        o.zero_grad()
        nn.functional.cross_entropy(m(x), y).backward()
        o.step()
    for r in range(2):
        for a, b in zip(got[r], model.parameters()):
            assert torch.allclose(a, b, atol=1e-6), mode


def _ddp_per_layer_job(rank, world):
    """Stock DistributedDataParallel + DistributedPerLayerOptimizer: every parameter is clipped to its own bound
    and finished inside backward; DDP's all-reduce carries the private gradients."""
    from torch.nn.parallel import DistributedDataParallel as DDP

    from opacus_b200.grad_sample import GradSampleModule
    from opacus_b200.optimizers import DistributedPerLayerOptimizer

    x, y = _data()
    base = _mlp()
    gsm = GradSampleModule(base, early_capture=True)
    ddp = DDP(gsm)
    bounds = [0.05 * (i + 1) for i, _ in enumerate(base.parameters())]
    opt = DistributedPerLayerOptimizer(torch.optim.SGD(base.parameters(), lr=0.5), noise_multiplier=0.0,
                                       max_grad_norm=bounds, expected_batch_size=4)
    xs, ys = x[rank::world], y[rank::world]
    for _ in range(2):
        opt.zero_grad()
        nn.functional.cross_entropy(ddp(xs), ys).backward()
        opt.step()
    assert opt.accumulated_iterations == 0
    return [p.detach().clone() for p in base.parameters()]


def test_ddp_per_layer_hooks_equal_single_process_per_layer_clipping():
    from opacus_b200.grad_sample import GradSampleModule
    from opacus_b200.optimizers import DPPerLayerOptimizer

    got = _run(_ddp_per_layer_job)
    x, y = _data()
    model = _mlp()
    gsm = GradSampleModule(model)
    bounds = [0.05 * (i + 1) for i, _ in enumerate(model.parameters())]
    opt = DPPerLayerOptimizer(torch.optim.SGD(model.parameters(), lr=0.5), noise_multiplier=0.0, max_grad_norm=bounds,
                              expected_batch_size=8)
    for _ in range(2):
        opt.zero_grad()
        nn.functional.cross_entropy(gsm(x), y).backward()
        opt.step()
    for r in range(2):
        for a, b in zip(got[r], model.parameters()):
            assert torch.allclose(a, b, atol=1e-6)


class _TPNet(nn.Module):
    def __init__(self, col, row):
        super().__init__()
        self.col, self.row = col, row
        self.ln = nn.LayerNorm(12)

    def forward(self, x):
        return self.ln(self.row(torch.tanh(self.col(x))))


def _tp_reference():
    torch.manual_seed(0)
    return _TPNet(nn.Linear(12, 16), nn.Linear(16, 12))


def _tp_job(rank, world):
    from opacus_b200.grad_sample import GradSampleModuleFastGradientClippingTP
    from opacus_b200.parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear, TensorParallelDPOptimizer
    from opacus_b200.utils.fast_gradient_clipping_utils import DPLossFastGradientClipping

    full = _tp_reference()
    net = _TPNet(ColumnParallelLinear.from_linear(full.col), RowParallelLinear.from_linear(full.row))
    net.ln.load_state_dict(full.ln.state_dict())
    x, _ = _data()
    x = x.reshape(4, 2, 12)
    results = {}
    for single_pass in (False, True):
        import copy

        model = copy.deepcopy(net)
        for p, q in zip(model.parameters(), net.parameters()):
            if getattr(q, "tp_sharded", False):
                p.tp_sharded = True
        gsm = GradSampleModuleFastGradientClippingTP(model, max_grad_norm=0.1, single_pass=single_pass)
        opt = TensorParallelDPOptimizer(torch.optim.SGD(model.parameters(), lr=0.5), noise_multiplier=0.0,
                                        max_grad_norm=0.1, expected_batch_size=4)
        crit = DPLossFastGradientClipping(gsm, opt, nn.MSELoss(), "mean")

        class PerSample:
            reduction = "mean"

            def __call__(self, out, tgt):
                per = (out - tgt).pow(2).flatten(1).mean(1)
                return per if self.reduction == "none" else per.mean()

        crit.criterion = PerSample()
        opt.zero_grad()
        crit(gsm(x), torch.zeros(4, 2, 12)).backward()
        opt.step()
        results[single_pass] = ({k: v.detach().clone() for k, v in model.state_dict().items()},
                                gsm.per_sample_gradient_norms.clone())
    return results


def _tp_noise_job(rank, world):
    """Both ranks seed alike (what every example does); a wide layer so that correlations are measurable."""
    from opacus_b200.parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear, TensorParallelDPOptimizer

    torch.manual_seed(0)
    full = _TPNet(nn.Linear(12, 256), nn.Linear(256, 12))
    net = _TPNet(ColumnParallelLinear.from_linear(full.col), RowParallelLinear.from_linear(full.row))
    torch.manual_seed(0)
    opt = TensorParallelDPOptimizer(torch.optim.SGD(net.parameters(), lr=1.0), noise_multiplier=2.0,
                                    max_grad_norm=0.5, expected_batch_size=1, loss_reduction="sum")
    out = {}
    for step in range(2):
        for p in net.parameters():
            p.summed_grad = torch.zeros_like(p)
        opt.add_noise()
        out[step] = {n: p.grad.detach().clone() for n, p in net.named_parameters()}
    return out


def test_tensor_parallel_noise_is_independent_between_shards_and_equal_on_replicas():
    got = _run(_tp_noise_job)
    std = 2.0 * 0.5
    for step in range(2):
        a, b = got[0][step], got[1][step]
        for name in ("col.weight", "row.weight"):          # shards: same shape on both ranks, different noise
            za, zb = a[name].flatten(), b[name].flatten()
            assert za.numel() >= 1536
            assert abs(float(za.std()) - std) < 0.1 * std and abs(float(zb.std()) - std) < 0.1 * std
            corr = float((za * zb).mean() / (za.std() * zb.std()))
            assert abs(corr) < 5.0 / za.numel() ** 0.5, (name, corr)
        for name in ("ln.weight", "ln.bias", "row.bias"):  # replicas: the same bits everywhere
            assert torch.equal(a[name], b[name]), name
            assert float(a[name].abs().sum()) > 0
    # a shard's noise also differs from step to step
    assert not torch.equal(got[0][0]["col.weight"], got[0][1]["col.weight"])


def _tp_secure_noise_job(rank, world):
    """secure_mode: every rank has its own ChaCha20 generator keyed from the OS pool."""
    from opacus_b200.parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear, TensorParallelDPOptimizer
    from opacus_b200.utils.secure_rng import SecureGenerator

    torch.manual_seed(0)
    full = _TPNet(nn.Linear(12, 256), nn.Linear(256, 12))
    net = _TPNet(ColumnParallelLinear.from_linear(full.col), RowParallelLinear.from_linear(full.row))
    opt = TensorParallelDPOptimizer(torch.optim.SGD(net.parameters(), lr=1.0), noise_multiplier=2.0, max_grad_norm=0.5,
                                    expected_batch_size=1, loss_reduction="sum", generator=SecureGenerator(),
                                    secure_mode=True)
    for p in net.parameters():
        p.summed_grad = torch.zeros_like(p)
    opt.add_noise()
    return {n: p.grad.detach().clone() for n, p in net.named_parameters()}


def test_tensor_parallel_secure_noise_shards_independent_replicas_equal():
    got = _run(_tp_secure_noise_job)
    a, b = got[0], got[1]
    for name in ("col.weight", "row.weight"):
        za, zb = a[name].flatten(), b[name].flatten()
        assert abs(float(za.std()) - 1.0) < 0.1 and abs(float(zb.std()) - 1.0) < 0.1
        corr = float((za * zb).mean() / (za.std() * zb.std()))
        assert abs(corr) < 5.0 / za.numel() ** 0.5, (name, corr)
    for name in ("ln.weight", "ln.bias", "row.bias"):      # drawn by the first rank of the group, broadcast
        assert torch.equal(a[name], b[name]) and float(a[name].abs().sum()) > 0


def test_tensor_parallel_ghost_matches_unsharded():
    from opacus_b200.grad_sample import GradSampleModuleFastGradientClipping
    from opacus_b200.optimizers import DPOptimizerFastGradientClipping
    from opacus_b200.utils.fast_gradient_clipping_utils import DPLossFastGradientClipping

    got = _run(_tp_job)
    model = _tp_reference()
    x, _ = _data()
    x = x.reshape(4, 2, 12)
    gsm = GradSampleModuleFastGradientClipping(model, max_grad_norm=0.1, single_pass=True)
    opt = DPOptimizerFastGradientClipping(torch.optim.SGD(model.parameters(), lr=0.5), noise_multiplier=0.0,
                                          max_grad_norm=0.1, expected_batch_size=4)

    class PerSample:
        reduction = "mean"

        def __call__(self, out, tgt):
            per = (out - tgt).pow(2).flatten(1).mean(1)
            return per if self.reduction == "none" else per.mean()

    crit = DPLossFastGradientClipping(gsm, opt, PerSample(), "mean")
    opt.zero_grad()
    crit(gsm(x), torch.zeros(4, 2, 12)).backward()
    norms = gsm.per_sample_gradient_norms.clone()
    opt.step()
    want = model.state_dict()
    for rank in range(2):
        for single_pass in (False, True):
            sd, n = got[rank][single_pass]
            assert torch.allclose(n, norms, rtol=1e-4, atol=1e-6), (rank, single_pass)
            assert torch.allclose(sd["col.weight"], want["col.weight"].chunk(2, 0)[rank], atol=1e-6)
            assert torch.allclose(sd["col.bias"], want["col.bias"].chunk(2, 0)[rank], atol=1e-6)
            assert torch.allclose(sd["row.weight"], want["row.weight"].chunk(2, 1)[rank], atol=1e-6)
            assert torch.allclose(sd["row.bias"], want["row.bias"], atol=1e-6)
            assert torch.allclose(sd["ln.weight"], want["ln.weight"], atol=1e-6)


def _sampler_job(rank, world):
    from opacus_b200.utils.uniform_sampler import DistributedUniformWithReplacementSampler

    s = DistributedUniformWithReplacementSampler(total_size=101, sample_rate=1.0, steps=1,
                                                 generator=torch.Generator().manual_seed(rank))
    return torch.cat(list(s))


def test_distributed_sampler_covers_dataset_once():
    parts = _run(_sampler_job)
    assert sorted(torch.cat(parts).tolist()) == list(range(101))


def _absent_rank_job(rank, world):
    """Rank 1 leaves between steps without joining the next collective; rank 0's
    collective must end with an error (short timeout) instead of hanging."""
    t = torch.ones(4)
    dist.all_reduce(t)
    if rank == 1:
        return "left"
    try:
        dist.all_reduce(t)
        return "no error"
    except Exception as e:  # gloo reports the missing peer / timeout
        return f"error: {type(e).__name__}"


def test_missing_rank_is_detected_by_timeout():
    res = _run(_absent_rank_job, timeout_s=5)
    assert res[1] == "left" and res[0].startswith("error")


# ------------------------------------------------------------------ tensor-parallel Llama + vocabulary-parallel loss
def _tiny_llama():
    from opacus_b200.models import Llama, LlamaConfig

    torch.manual_seed(3)
    return Llama(LlamaConfig(vocab_size=96, d_model=32, n_layers=2, n_heads=4, n_kv_heads=2, ffn_dim=64,
                             tie_embeddings=False))


def _llama_ids():
    g = torch.Generator().manual_seed(11)
    return torch.randint(0, 96, (3, 9), generator=g)


def _tp_llama_job(rank, world):
    from opacus_b200.grad_sample import GradSampleModuleFastGradientClippingTP
    from opacus_b200.parallel.tensor_parallel import (TensorParallelDPOptimizer, VocabParallelCrossEntropy,
                                                      parallelize_llama)
    from opacus_b200.utils.fast_gradient_clipping_utils import DPLossFastGradientClipping

    model = parallelize_llama(_tiny_llama())
    ids = _llama_ids()
    gsm = GradSampleModuleFastGradientClippingTP(model, max_grad_norm=0.05, single_pass=True)
    opt = TensorParallelDPOptimizer(torch.optim.SGD(model.parameters(), lr=0.5), noise_multiplier=0.0,
                                    max_grad_norm=0.05, expected_batch_size=3)
    crit = DPLossFastGradientClipping(gsm, opt, VocabParallelCrossEntropy(), "mean")
    opt.zero_grad()
    logits = gsm(ids[:, :-1])
    loss = crit(logits.flatten(0, 1), ids[:, 1:].reshape(-1), shape=(3, 8))
    value = loss.item()
    loss.backward()
    opt.step()
    return value, gsm.per_sample_gradient_norms.clone(), {k: v.detach().clone() for k, v in model.state_dict().items()}


def test_tensor_parallel_llama_matches_unsharded():
    from opacus_b200.grad_sample import GradSampleModuleFastGradientClipping
    from opacus_b200.optimizers import DPOptimizerFastGradientClipping
    from opacus_b200.utils.fast_gradient_clipping_utils import DPLossFastGradientClipping

    got = _run(_tp_llama_job, timeout_s=120)
    model = _tiny_llama()
    ids = _llama_ids()
    gsm = GradSampleModuleFastGradientClipping(model, max_grad_norm=0.05, single_pass=True)
    opt = DPOptimizerFastGradientClipping(torch.optim.SGD(model.parameters(), lr=0.5), noise_multiplier=0.0,
                                          max_grad_norm=0.05, expected_batch_size=3)
    crit = DPLossFastGradientClipping(gsm, opt, nn.CrossEntropyLoss(), "mean")
    opt.zero_grad()
    loss = crit(gsm(ids[:, :-1]).flatten(0, 1), ids[:, 1:].reshape(-1), shape=(3, 8))
    value = loss.item()
    loss.backward()
    norms = gsm.per_sample_gradient_norms.clone()
    opt.step()
    want = model.state_dict()
    for rank in range(2):
        v, n, sd = got[rank]
        assert abs(v - value) < 1e-5
        assert torch.allclose(n, norms, rtol=1e-4, atol=1e-6), rank
        for name, full in want.items():
            mine = sd[name]
            if mine.shape == full.shape:
                ref = full
            elif mine.shape[0] != full.shape[0]:
                ref = full.chunk(2, 0)[rank]          # column-parallel: output features split
            else:
                ref = full.chunk(2, 1)[rank]          # row-parallel: input features split
            assert torch.allclose(mine, ref, atol=2e-6), (rank, name)


def _llama_ids4():
    g = torch.Generator().manual_seed(12)
    return torch.randint(0, 96, (4, 9), generator=g)


def _tp_sp_llama_job(rank, world):
    from opacus_b200.grad_sample import GradSampleModuleFastGradientClippingTP
    from opacus_b200.parallel.tensor_parallel import (TensorParallelDPOptimizer, VocabParallelCrossEntropy,
                                                      parallelize_llama)
    from opacus_b200.utils.fast_gradient_clipping_utils import DPLossFastGradientClipping

    model = parallelize_llama(_tiny_llama(), sequence_parallel=True)
    ids = _llama_ids4()
    gsm = GradSampleModuleFastGradientClippingTP(model, max_grad_norm=0.05, single_pass=True)
    opt = TensorParallelDPOptimizer(torch.optim.SGD(model.parameters(), lr=0.5), noise_multiplier=0.0,
                                    max_grad_norm=0.05, expected_batch_size=4)
    crit = DPLossFastGradientClipping(gsm, opt, VocabParallelCrossEntropy(), "mean")
    out = []
    for _ in range(2):                       # two steps: buffers and flags are reused
        opt.zero_grad()
        logits = gsm(ids[:, :-1])
        loss = crit(logits.flatten(0, 1), ids[:, 1:].reshape(-1), shape=(4, 8))
        value = loss.item()
        loss.backward()
        norms = gsm.per_sample_gradient_norms.clone()
        opt.step()
        out.append((value, norms))
    return out, {k: v.detach().clone() for k, v in model.state_dict().items()}


def test_sequence_parallel_llama_matches_unsharded():
    """Activations sharded over samples between the tensor-parallel blocks: same losses, per-sample norms
    and updated weights as the unsharded model (embedding / norm weights get their partial sums all-reduced)."""
    from opacus_b200.grad_sample import GradSampleModuleFastGradientClipping
    from opacus_b200.optimizers import DPOptimizerFastGradientClipping
    from opacus_b200.utils.fast_gradient_clipping_utils import DPLossFastGradientClipping

    got = _run(_tp_sp_llama_job, timeout_s=180)
    model = _tiny_llama()
    ids = _llama_ids4()
    gsm = GradSampleModuleFastGradientClipping(model, max_grad_norm=0.05, single_pass=True)
    opt = DPOptimizerFastGradientClipping(torch.optim.SGD(model.parameters(), lr=0.5), noise_multiplier=0.0,
                                          max_grad_norm=0.05, expected_batch_size=4)
    crit = DPLossFastGradientClipping(gsm, opt, nn.CrossEntropyLoss(), "mean")
    ref = []
    for _ in range(2):
        opt.zero_grad()
        loss = crit(gsm(ids[:, :-1]).flatten(0, 1), ids[:, 1:].reshape(-1), shape=(4, 8))
        value = loss.item()
        loss.backward()
        ref.append((value, gsm.per_sample_gradient_norms.clone()))
        opt.step()
    want = model.state_dict()
    for rank in range(2):
        steps, sd = got[rank]
        for (v, n), (rv, rn) in zip(steps, ref):
            assert abs(v - rv) < 1e-5
            assert torch.allclose(n, rn, rtol=1e-4, atol=1e-6), rank
        for name, full in want.items():
            mine = sd[name]
            if mine.shape == full.shape:
                refw = full
            elif mine.shape[0] != full.shape[0]:
                refw = full.chunk(2, 0)[rank]
            else:
                refw = full.chunk(2, 1)[rank]
            assert torch.allclose(mine, refw, atol=3e-6), (rank, name)
