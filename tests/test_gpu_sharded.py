"""The sharded data-parallel engine on one GPU (world size 1) against the plain
ghost path, and its fused step kernel against torch.optim."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.nn as nn
from torch.utils.data import DataLoader, TensorDataset

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pg():
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29541")
    if not dist.is_initialized():
        dist.init_process_group("nccl", rank=0, world_size=1)
    yield
    dist.destroy_process_group()


def _model():
    from opacus_b200.models import Llama, LlamaConfig

    torch.manual_seed(0)
    return Llama(LlamaConfig(vocab_size=512, d_model=128, n_layers=2, n_heads=4, n_kv_heads=2, ffn_dim=256)).cuda()


def _private(module, mode, sigma, opt_cls=torch.optim.AdamW, **kw):
    from opacus_b200 import PrivacyEngine

    inner = module.module if hasattr(module, "module") else module
    opt = opt_cls(inner.parameters(), lr=1e-2, **kw)
    dl = DataLoader(TensorDataset(torch.zeros(32, 1)), batch_size=4)
    pe = PrivacyEngine(accountant="rdp")
    return pe.make_private(module=module, optimizer=opt, criterion=nn.CrossEntropyLoss(), data_loader=dl,
                           noise_multiplier=sigma, max_grad_norm=0.5, grad_sample_mode=mode, poisson_sampling=False)


def _step(m, opt, crit, ids):
    opt.zero_grad(set_to_none=True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        logits = m(ids[:, :-1])
    loss = crit(logits.float().flatten(0, 1), ids[:, 1:].reshape(-1), shape=(ids.shape[0], ids.shape[1] - 1))
    loss.backward()
    opt.step()
    return loss.item()


@pytest.mark.parametrize("opt_cls,kw", [(torch.optim.AdamW, {}), (torch.optim.SGD, {"momentum": 0.9})])
def test_sharded_engine_world1_matches_fp32_master_reference(pg, opt_cls, kw):
    from opacus_b200.parallel.sharded import ShardedDataParallel
    from opacus_b200.ops import _cuda

    ids = torch.randint(0, 512, (4, 129), device="cuda")
    eng = ShardedDataParallel(_model())
    m, opt, crit, _ = _private(eng, "ghost_fsdp", 0.0, opt_cls, **kw)
    norms = []
    for _ in range(3):
        _step(m, opt, crit, ids)
        norms.append(m.per_sample_gradient_norms.clone())
    torch.cuda.synchronize()
    _cuda.check_status()
    got = eng.full_precision_state_dict()

    # reference: the same bf16-compute / fp32-master recipe spelled out with torch ops
    ref = _model()
    master = {n: p.detach().clone().float() for n, p in ref.named_parameters()}
    ref = ref.bfloat16()
    from opacus_b200.grad_sample import GradSampleModuleFastGradientClipping
    from opacus_b200.optimizers import DPOptimizerFastGradientClipping
    from opacus_b200.utils.fast_gradient_clipping_utils import DPLossFastGradientClipping

    shadow = [nn.Parameter(v.clone()) for v in master.values()]
    torch_opt = opt_cls(shadow, lr=1e-2, **kw)
    gsm = GradSampleModuleFastGradientClipping(ref, max_grad_norm=0.5, single_pass=True)
    dpo = DPOptimizerFastGradientClipping(torch.optim.SGD(ref.parameters(), lr=0.0), noise_multiplier=0.0,
                                          max_grad_norm=0.5, expected_batch_size=4, fused_step=False)
    crit2 = DPLossFastGradientClipping(gsm, dpo, nn.CrossEntropyLoss(), "mean")
    for it in range(3):
        for p in ref.parameters():
            p.grad = None
        logits = gsm(ids[:, :-1])
        crit2(logits.float().flatten(0, 1), ids[:, 1:].reshape(-1), shape=(4, 128)).backward()
        assert torch.allclose(gsm.per_sample_gradient_norms, norms[it], rtol=2e-2), (it, gsm.per_sample_gradient_norms, norms[it])
        seen = set()
        for (n, p), s in zip(ref.named_parameters(), shadow):
            s.grad = p.grad.float() / 4
        torch_opt.step()
        for (n, p), s in zip(ref.named_parameters(), shadow):
            p.data.copy_(s.data.to(torch.bfloat16))
    for (n, _), s in zip(ref.named_parameters(), shadow):
        a, b = got[n], s.detach()
        assert ((a - b).norm() / (b.norm() + 1e-12)).item() < 2e-2, (n, (a - b).abs().max())


def test_sharded_engine_noise_and_virtual_steps(pg):
    from opacus_b200.parallel.sharded import ShardedDataParallel

    ids = torch.randint(0, 512, (4, 65), device="cuda")
    eng = ShardedDataParallel(_model())
    before = eng.master.clone()
    m, opt, crit, _ = _private(eng, "ghost_fsdp", 100.0, torch.optim.SGD)
    opt.signal_skip_step(True)
    _step(m, opt, crit, ids)                       # accumulate only
    assert torch.equal(eng.master, before)
    g1 = eng.flat_grad().clone()
    opt.signal_skip_step(False)
    _step(m, opt, crit, ids)                       # second physical batch + the update
    torch.cuda.synchronize()
    delta = (eng.master - before) / 1e-2 * 4        # = -(sum of clipped grads + noise)
    assert abs(delta.std().item() - 100.0 * 0.5) / 50.0 < 0.05
    assert g1.abs().sum() > 0


def test_piecewise_step_equals_single_launch(pg):
    """The flat space cut into pieces (stepped on a side stream beside the clipped-sum GEMMs) gives the weights of
    the one-launch step, noise included: the draw of an element depends on its index only."""
    from opacus_b200.parallel.sharded import ShardedDataParallel

    ids = torch.randint(0, 512, (4, 129), device="cuda")
    results = []
    for pieces in (1, 5):
        eng = ShardedDataParallel(_model(), step_pieces=pieces)
        gen = torch.Generator(device="cuda").manual_seed(11)
        from opacus_b200 import PrivacyEngine

        opt = torch.optim.AdamW(eng.module.parameters(), lr=1e-2)
        dl = DataLoader(TensorDataset(torch.zeros(32, 1)), batch_size=4)
        m, opt, crit, _ = PrivacyEngine(accountant="rdp").make_private(
            module=eng, optimizer=opt, criterion=nn.CrossEntropyLoss(), data_loader=dl, noise_multiplier=1.0,
            max_grad_norm=0.5, grad_sample_mode="ghost_fsdp", poisson_sampling=False, noise_generator=gen)
        for _ in range(3):
            _step(m, opt, crit, ids)
        torch.cuda.synchronize()
        assert (eng.last_step_launches == 1) == (pieces == 1)
        results.append(eng.full_precision_state_dict())
    for k in results[0]:
        a, b = results[0][k], results[1][k]
        assert ((a - b).norm() / (a.norm() + 1e-12)).item() < 1e-4, k


def test_engine_param_groups_with_own_lr_and_weight_decay(pg):
    """Two parameter groups (decay / no decay, different learning rates) against torch.optim.AdamW on fp32 copies
    fed with the engine's own clipped sums."""
    from opacus_b200.parallel.sharded import ShardedDataParallel

    ids = torch.randint(0, 512, (4, 65), device="cuda")
    model = _model()
    eng = ShardedDataParallel(model)
    decay = [p for n, p in model.named_parameters() if p.dim() >= 2]
    no_decay = [p for n, p in model.named_parameters() if p.dim() < 2]
    groups = [{"params": decay, "weight_decay": 0.1, "lr": 1e-2}, {"params": no_decay, "weight_decay": 0.0, "lr": 3e-2}]
    from opacus_b200 import PrivacyEngine

    opt = torch.optim.AdamW(groups)
    dl = DataLoader(TensorDataset(torch.zeros(32, 1)), batch_size=4)
    m, opt, crit, _ = PrivacyEngine(accountant="rdp").make_private(
        module=eng, optimizer=opt, criterion=nn.CrossEntropyLoss(), data_loader=dl, noise_multiplier=0.0,
        max_grad_norm=0.5, grad_sample_mode="ghost_fsdp", poisson_sampling=False)
    start = eng.full_precision_state_dict()
    names = {id(p): n for n, p in model.named_parameters()}
    shadow = {n: nn.Parameter(v.clone()) for n, v in start.items()}
    ref = torch.optim.AdamW([{"params": [shadow[names[id(p)]] for p in decay], "weight_decay": 0.1, "lr": 1e-2},
                             {"params": [shadow[names[id(p)]] for p in no_decay], "weight_decay": 0.0, "lr": 3e-2}])
    for _ in range(2):
        opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            logits = m(ids[:, :-1])
        crit(logits.float().flatten(0, 1), ids[:, 1:].reshape(-1), shape=(4, 64)).backward()
        torch.cuda.synchronize()
        for n, p in model.named_parameters():          # the sums the step is about to consume
            shadow[n].grad = p._dp_grad_out.detach().clone() / 4
        opt.step()
        ref.step()
    got = eng.full_precision_state_dict()
    for n in got:
        assert torch.allclose(got[n], shadow[n].detach(), rtol=1e-4, atol=1e-6), (n, (got[n] - shadow[n]).abs().max())


def test_engine_checkpoint_resume(pg, tmp_path):
    """k steps, save_checkpoint, fresh engine, load_checkpoint, k steps == 2k steps in one go; the optimiser file has
    torch.optim's layout; loading weights through the engine is not undone by the next step."""
    from opacus_b200 import PrivacyEngine
    from opacus_b200.parallel.sharded import ShardedDataParallel

    ids = torch.randint(0, 512, (4, 65), device="cuda")

    def fresh(shift=0.0):
        model = _model()
        if shift:
            with torch.no_grad():
                for p in model.parameters():
                    p.add_(shift)
        eng = ShardedDataParallel(model)
        opt = torch.optim.AdamW(model.parameters(), lr=1e-2)
        dl = DataLoader(TensorDataset(torch.zeros(32, 1)), batch_size=4)
        pe = PrivacyEngine(accountant="rdp")
        m, opt, crit, _ = pe.make_private(module=eng, optimizer=opt, criterion=nn.CrossEntropyLoss(), data_loader=dl,
                                          noise_multiplier=0.0, max_grad_norm=0.5, grad_sample_mode="ghost_fsdp",
                                          poisson_sampling=False)
        return pe, eng, m, opt, crit

    def steps(m, opt, crit, n):
        for _ in range(n):
            opt.zero_grad(set_to_none=True)
            with torch.autocast("cuda", dtype=torch.bfloat16):
                logits = m(ids[:, :-1])
            crit(logits.float().flatten(0, 1), ids[:, 1:].reshape(-1), shape=(4, 64)).backward()
            opt.step()

    pe, eng, m, opt, crit = fresh()
    steps(m, opt, crit, 2)
    path = str(tmp_path / "ckpt.pt")
    pe.save_checkpoint(path=path, module=m, optimizer=opt)
    steps(m, opt, crit, 2)
    want = eng.full_precision_state_dict()

    saved = torch.load(path, weights_only=False)
    osd = saved["optimizer_state_dict"]
    assert set(osd) == {"state", "param_groups"} and len(osd["state"]) == len(list(eng.module.parameters()))
    first = osd["state"][0]
    assert set(first) == {"step", "exp_avg", "exp_avg_sq"} and float(first["step"]) == 2.0
    assert first["exp_avg"].dtype == torch.float32 and first["exp_avg"].shape == next(eng.module.parameters()).shape
    assert all(v.dtype == torch.float32 for k, v in saved["module_state_dict"].items() if v.is_floating_point())

    pe2, eng2, m2, opt2, crit2 = fresh(shift=0.5)
    pe2.load_checkpoint(path=path, module=m2, optimizer=opt2)
    steps(m2, opt2, crit2, 2)
    got = eng2.full_precision_state_dict()
    for k in want:
        assert ((got[k] - want[k]).norm() / (want[k].norm() + 1e-12)).item() < 1e-4, k

    # weights loaded into the wrapped module directly survive the next step too
    pe3, eng3, m3, opt3, crit3 = fresh(shift=0.25)
    eng3.module.load_state_dict({k[len("_module."):]: v for k, v in saved["module_state_dict"].items()})
    steps(m3, opt3, crit3, 1)
    moved = eng3.full_precision_state_dict()
    k0 = next(iter(moved))
    assert (moved[k0] - saved["module_state_dict"]["_module." + k0].cuda()).abs().max() < 0.1


def test_engine_state_loads_a_torch_optim_file(pg):
    """An optimiser file written by plain torch.optim over the same parameters loads into the engine."""
    from opacus_b200.optimizers import FSDPOptimizerFastGradientClipping
    from opacus_b200.parallel.sharded import ShardedDataParallel

    plain = _model()
    topt = torch.optim.AdamW(plain.parameters(), lr=1e-2)
    for p in plain.parameters():
        p.grad = torch.randn_like(p)
    topt.step()
    file = topt.state_dict()
    model = _model()
    eng = ShardedDataParallel(model)
    dpo = FSDPOptimizerFastGradientClipping(torch.optim.AdamW(model.parameters(), lr=5e-3), noise_multiplier=0.0,
                                            max_grad_norm=1.0, expected_batch_size=4, engine=eng)
    dpo.load_state_dict(file)
    assert eng._steps == 1 and dpo.param_groups[0]["lr"] == 1e-2
    back = dpo.state_dict()
    for idx, entry in file["state"].items():
        assert torch.equal(back["state"][idx]["exp_avg"], entry["exp_avg"].float())
        assert torch.equal(back["state"][idx]["exp_avg_sq"], entry["exp_avg_sq"].float())


def test_engine_secure_mode_noise_comes_from_the_optimizer_generator(pg):
    """With secure_mode the engine adds host-generated noise (five-draw rule) to the stripes it owns and runs the
    kernel without its own draw: the update then has the std of one draw of sigma * C."""
    from opacus_b200.parallel.sharded import ShardedDataParallel

    ids = torch.randint(0, 512, (4, 65), device="cuda")
    eng = ShardedDataParallel(_model(), step_pieces=3)
    before = eng.master.clone()
    m, opt, crit, _ = _private(eng, "ghost_fsdp", 100.0, torch.optim.SGD)
    opt.secure_mode = True
    opt.generator = torch.Generator(device="cuda").manual_seed(3)
    _step(m, opt, crit, ids)
    torch.cuda.synchronize()
    delta = (eng.master - before) / 1e-2 * 4
    assert abs(delta.std().item() - 100.0 * 0.5) / 50.0 < 0.05


def _wide_model():
    from opacus_b200.models import Llama, LlamaConfig

    torch.manual_seed(0)
    return Llama(LlamaConfig(vocab_size=512, d_model=256, n_layers=2, n_heads=4, n_kv_heads=2, ffn_dim=512)).cuda()


def test_parameter_sharding_equals_replicated_engine(pg, tmp_path):
    """shard_params=True (row-sharded Linear weights: fused all-gather -> GEMM forward, layer-by-layer reduce-scatter +
    step) trains like the replicated layout, and its checkpoint holds whole fp32 weights."""
    from opacus_b200 import PrivacyEngine
    from opacus_b200.parallel.param_sharding import ShardedLinear
    from opacus_b200.parallel.sharded import ShardedDataParallel

    ids = torch.randint(0, 512, (4, 129), device="cuda")
    results = {}
    for shard in (False, True):
        model = _wide_model()
        eng = ShardedDataParallel(model, shard_params=shard)
        n_sharded = sum(isinstance(m, ShardedLinear) for m in model.modules())
        assert (n_sharded > 0) == shard
        if shard:
            assert n_sharded == 2 * 5                      # q, o, gate, up, down of both blocks; k / v are too narrow
        m, opt, crit, _ = _private(eng, "ghost_fsdp", 0.0, torch.optim.AdamW, weight_decay=0.05)
        for _ in range(3):
            _step(m, opt, crit, ids)
        torch.cuda.synchronize()
        results[shard] = (eng.full_precision_state_dict(), m.per_sample_gradient_norms.clone(), eng, m, opt)
    a, b = results[False][0], results[True][0]
    assert set(a) == set(b)
    assert torch.allclose(results[False][1], results[True][1], rtol=2e-2)
    for k in a:
        assert a[k].shape == b[k].shape, k
        assert ((a[k] - b[k]).norm() / (a[k].norm() + 1e-12)).item() < 2e-2, k
    # checkpoint of the sharded layout: whole fp32 weights under the model's own keys, torch.optim optimizer layout
    _, _, eng, m, opt = results[True]
    sd = m.state_dict()
    key = "_module.layers.0.self_attn.q_proj.weight"
    assert sd[key].shape == (256, 256) and sd[key].dtype == torch.float32
    osd = opt.state_dict()
    shapes = {tuple(v["exp_avg"].shape) for v in osd["state"].values()}
    assert (512, 256) in shapes and (256, 512) in shapes
    # a fresh sharded engine resumes from it
    model2 = _wide_model()
    with torch.no_grad():
        for p in model2.parameters():
            p.add_(0.3)
    eng2 = ShardedDataParallel(model2, shard_params=True)
    m2, opt2, crit2, _ = _private(eng2, "ghost_fsdp", 0.0, torch.optim.AdamW, weight_decay=0.05)
    m2.load_state_dict(sd)
    opt2.load_state_dict(osd)
    _step(m, opt, crit, ids)
    _step(m2, opt2, crit2, ids)
    torch.cuda.synchronize()
    x, y = eng.full_precision_state_dict(), eng2.full_precision_state_dict()
    for k in x:
        assert ((x[k] - y[k]).norm() / (x[k].norm() + 1e-12)).item() < 1e-3, k


def test_engine_serves_hooks_mode_data_parallel(pg):
    """DistributedDPOptimizer on top of the engine (fp32 compute weights) equals the plain DPOptimizer."""
    import copy

    from opacus_b200 import PrivacyEngine
    from opacus_b200.parallel.sharded import ShardedDataParallel

    torch.manual_seed(0)
    base = nn.Sequential(nn.Linear(32, 64), nn.ReLU(), nn.LayerNorm(64), nn.Linear(64, 8)).cuda()
    twin = copy.deepcopy(base)
    x = torch.randn(16, 32, device="cuda")
    y = torch.randint(0, 8, (16,), device="cuda")
    dl = DataLoader(TensorDataset(torch.zeros(64, 1)), batch_size=16)

    eng = ShardedDataParallel(base, param_dtype=torch.float32)
    m1, o1, _ = PrivacyEngine(accountant="rdp").make_private(
        module=eng, optimizer=torch.optim.SGD(base.parameters(), lr=0.1, momentum=0.9), data_loader=dl,
        noise_multiplier=0.0, max_grad_norm=0.3, poisson_sampling=False)
    m2, o2, _ = PrivacyEngine(accountant="rdp").make_private(
        module=twin, optimizer=torch.optim.SGD(twin.parameters(), lr=0.1, momentum=0.9), data_loader=dl,
        noise_multiplier=0.0, max_grad_norm=0.3, poisson_sampling=False)
    assert type(o1).__name__ == "DistributedDPOptimizer" and o1.engine is eng
    for _ in range(3):
        for m, o in ((m1, o1), (m2, o2)):
            o.zero_grad()
            nn.functional.cross_entropy(m(x), y).backward()
            o.step()
    torch.cuda.synchronize()
    for a, b in zip(base.parameters(), twin.parameters()):
        assert torch.allclose(a, b, rtol=1e-4, atol=1e-5), (a - b).abs().max()


@pytest.mark.gpu
def test_peer_norm_reducer_single_rank():
    from opacus_b200.ops import _cuda
    from opacus_b200.parallel import symm

    red = symm.PeerNormReducer(torch.device("cuda", 0), capacity=256)
    a, b = torch.rand(200, device="cuda"), torch.rand(200, device="cuda")
    for _ in range(3):          # both slot parities
        total, clip = red(a, b, 1.5)
        assert torch.equal(total, a + b)
        torch.testing.assert_close(clip, (1.5 / ((a + b).sqrt() + 1e-6)).clamp(max=1.0))
    total, _ = red(None, b, 1.0)
    assert torch.equal(total, b)
    big = torch.rand(300, device="cuda")                 # longer than the capacity: the buffers grow
    total, _ = red(big, None, 1.0)
    assert red.capacity >= 300 and torch.equal(total, big)
    _cuda.check_status()


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (384, 520, 200), (1024, 2048, 1024)])
def test_gemm_nt_kernel(M, N, K):
    from opacus_b200.ops import _cuda
    from opacus_b200.parallel.fused_tp import gemm_nt

    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    ref = a.float() @ b.float().t()
    out = gemm_nt(a, b)
    assert (out.float() - ref).abs().max() <= 1e-2 * ref.abs().max()
    _cuda.check_status()


@pytest.mark.gpu
def test_fused_collective_gemms_single_rank():
    """One-rank group: the copier / slot / flag machinery runs, the collective is the identity."""
    from opacus_b200.ops import _cuda
    from opacus_b200.parallel.fused_tp import AllGatherGemm, GemmReduceScatter

    torch.manual_seed(0)
    dev = torch.device("cuda", 0)
    x = torch.randn(512, 320, device=dev).bfloat16()
    w = torch.randn(768, 320, device=dev).bfloat16()
    ref = x.float() @ w.float().t()
    ag = AllGatherGemm(512, 320, dev, gather="a")
    for _ in range(2):
        ag.shard.copy_(x)
        y = ag(w)
        assert (y.float() - ref).abs().max() <= 1e-2 * ref.abs().max()
        assert torch.equal(ag.full, x)
    agb = AllGatherGemm(768, 320, dev, gather="b")
    agb.shard.copy_(w)
    y = agb(x)
    assert (y.float() - ref).abs().max() <= 1e-2 * ref.abs().max()
    rs = GemmReduceScatter(512, 768, dev)
    for _ in range(3):
        y = rs(x, w)
        assert (y.float() - ref).abs().max() <= 1e-2 * ref.abs().max()
    _cuda.check_status()


@pytest.mark.gpu
def test_bounded_wait_runs_out_and_is_reported():
    """A rank whose peer never raises its flag: the kernel gives up after its time limit, the host gets
    CommTimeoutError on the next check, and the CUDA context keeps working."""
    from opacus_b200.ops import _cuda
    from opacus_b200.utils.errors import CommTimeoutError

    C = _cuda.load()
    dev = torch.device("cuda", 0)
    _cuda.check_status()
    slots = [torch.zeros(2 * 2 * 64, device=dev) for _ in range(2)]          # "rank 1" is a buffer nobody drives
    flags = [torch.zeros(64, dtype=torch.int32, device=dev) for _ in range(2)]
    part = torch.rand(8, device=dev)
    C.norm_allreduce_clip([s.data_ptr() for s in slots], [f.data_ptr() for f in flags], part, None, 8, 64, 0, 0, 1,
                          1.0, dev)
    torch.cuda.synchronize()                    # returns: the wait is limited to about two seconds
    with pytest.raises(CommTimeoutError):
        _cuda.check_status()
    _cuda.check_status()                        # the report is consumed
    x = torch.full((1024,), 2.0, device=dev)
    assert x.sum().item() == 2048.0             # the context is alive
    red_total, _ = C.norm_allreduce_clip([slots[0].data_ptr()], [flags[0].data_ptr()], part, None, 8, 64, 0, 32, 1, 1.0, dev)
    torch.cuda.synchronize()
    assert torch.equal(red_total, part)
    _cuda.check_status()


def test_step_kernel_noise_ranges_for_tensor_parallel_shards():
    """Elements at or beyond ``noise_split`` draw from the Philox range shifted by ``noise_shift``: below the split two
    tensor-parallel ranks see the same noise, beyond it independent noise -- the draw of index ``i + shift``."""
    from opacus_b200.ops import _cuda

    C = _cuda.load()
    dev = torch.device("cuda")
    n, split, shift = 8192, 2048, 4096

    def noise(length, split_at, shift_by):
        grad = torch.zeros(length, device=dev)
        param = torch.zeros(length, device=dev, dtype=torch.bfloat16)
        flags = torch.zeros(64, device=dev, dtype=torch.int32)
        master = torch.zeros(length, device=dev)
        # plain SGD, lr 1, no momentum: master = -(0 + noise) * inv_scale
        C.sharded_dp_step([grad.data_ptr()], [param.data_ptr()], [flags.data_ptr()], master, None, None, 0, length, 0,
                          True, 1, 0, False, False, 1.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 1.0, 1.0, 1.0, 1.0, 1234, 0,
                          split_at, shift_by)
        torch.cuda.synchronize()
        return -master

    base = noise(n, 0, 0)
    moved = noise(n // 2, split, shift)
    assert torch.equal(moved[:split], base[:split])
    assert torch.equal(moved[split:], base[split + shift: n // 2 + shift])
    assert not torch.equal(moved[split:], base[split: n // 2])
    assert 0.9 < float(base.std()) < 1.1
    _cuda.check_status()

