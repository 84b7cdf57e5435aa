"""The ChaCha20 generator behind ``secure_mode`` (``opacus_b200/utils/secure_rng.py``, ``csrc/secure_rng.cu``)."""
import numpy as np
import pytest
import torch
import torch.nn as nn
from torch.utils.data import DataLoader, TensorDataset

from opacus_b200 import PrivacyEngine
from opacus_b200.utils.secure_rng import (SecureGenerator, SecureRandomSampler, chacha20_blocks, rfc7539_block_check)

KEY = bytes(range(32))


def test_block_function_matches_rfc7539_vector():
    key = np.frombuffer(KEY, dtype="<u4")
    block = chacha20_blocks(key, 0x4A000000, 1 | (0x09000000 << 32), 1)[0]
    assert rfc7539_block_check(block)


def test_stream_is_consumed_once_and_is_reproducible():
    a, b = SecureGenerator(KEY), SecureGenerator(KEY)
    first, second = a.words(16), a.words(20)
    both = b.words(48)                          # blocks 0, 1, 2
    assert torch.equal(first, both[:16]) and torch.equal(second, both[16:36])
    assert a.counter == 3 and b.counter == 3
    other = SecureGenerator(bytes(range(1, 33))).words(16)
    assert not torch.equal(other, first)
    assert SecureGenerator().key.tobytes() != SecureGenerator().key.tobytes()      # keyed from the OS pool


def test_uniform_and_normal_statistics():
    g = SecureGenerator(KEY)
    u = g.rand(200_000)
    assert 0.0 <= u.min() and u.max() < 1.0 and abs(u.mean() - 0.5) < 5e-3 and abs(u.var() - 1 / 12) < 2e-3
    for draws in (1, 4):
        z = g.gaussian_like(torch.empty(400_000), 2.5, draws=draws)
        assert abs(z.mean()) < 2e-2 and abs(z.std() - 2.5) < 2e-2
        kurt = ((z / 2.5) ** 4).mean()
        assert abs(kurt - 3.0) < 0.1
    assert torch.equal(g.gaussian_like(torch.empty(7, 3), 0.0), torch.zeros(7, 3))
    assert g.gaussian_like(torch.empty(5, dtype=torch.float64), 1.0).dtype == torch.float64


def test_permutation_sampler():
    g = SecureGenerator(KEY)
    perm = g.randperm(1000)
    assert sorted(perm.tolist()) == list(range(1000)) and perm.tolist() != list(range(1000))
    data = list(range(50))
    assert sorted(SecureRandomSampler(data, g)) == data
    drawn = list(SecureRandomSampler(data, g, replacement=True, num_samples=80))
    assert len(drawn) == 80 and all(0 <= i < 50 for i in drawn)


def test_secure_mode_trains_with_the_own_generator():
    """Without torchcsprng, ``secure_mode=True`` runs on the ChaCha20 generator: Poisson sampling and noise."""
    pytest.importorskip("opacus_b200")
    try:
        import torchcsprng  # noqa: F401
        pytest.skip("torchcsprng is installed; the engine uses it")
    except ImportError:
        pass
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(10, 8), nn.ReLU(), nn.Linear(8, 2))
    data = TensorDataset(torch.randn(256, 10), torch.randint(0, 2, (256,)))
    engine = PrivacyEngine(accountant="rdp", secure_mode=True)
    assert isinstance(engine.secure_rng, SecureGenerator)
    before = torch.cat([p.detach().flatten().clone() for p in model.parameters()])
    model, opt, loader = engine.make_private(module=model, optimizer=torch.optim.SGD(model.parameters(), lr=0.1),
                                             data_loader=DataLoader(data, batch_size=32), noise_multiplier=1.0,
                                             max_grad_norm=1.0)
    assert opt.generator is engine.secure_rng and opt.secure_mode
    sizes = []
    for x, y in loader:
        sizes.append(len(x))
        opt.zero_grad()
        nn.functional.cross_entropy(model(x), y).backward()
        opt.step()
    assert len(set(sizes)) > 1                      # Poisson batches vary in size
    after = torch.cat([p.detach().flatten() for p in model.parameters()])
    assert torch.isfinite(after).all() and not torch.equal(before, after)
    assert engine.secure_rng.counter > 0
    with pytest.raises(ValueError):
        engine.make_private(module=nn.Linear(10, 2), optimizer=torch.optim.SGD(nn.Linear(10, 2).parameters(), lr=0.1),
                            data_loader=DataLoader(data, batch_size=32), noise_multiplier=1.0, max_grad_norm=1.0,
                            noise_generator=torch.Generator())


def test_secure_mode_without_poisson_sampling_shuffles_from_the_generator():
    try:
        import torchcsprng  # noqa: F401
        pytest.skip("torchcsprng is installed; the engine uses it")
    except ImportError:
        pass
    model = nn.Linear(4, 2)
    data = TensorDataset(torch.arange(64, dtype=torch.float32).repeat(4, 1).t().contiguous(), torch.zeros(64, dtype=torch.long))
    engine = PrivacyEngine(accountant="rdp", secure_mode=True)
    model, opt, loader = engine.make_private(module=model, optimizer=torch.optim.SGD(model.parameters(), lr=0.1),
                                             data_loader=DataLoader(data, batch_size=16, shuffle=True),
                                             noise_multiplier=1.0, max_grad_norm=1.0, poisson_sampling=False)
    seen = torch.cat([x[:, 0] for x, _ in loader]).long().tolist()
    assert sorted(seen) == list(range(64)) and seen != list(range(64))
    assert isinstance(loader.batch_sampler.sampler, SecureRandomSampler)


@pytest.mark.gpu
def test_cuda_kernel_computes_the_same_stream():
    g_cpu, g_gpu = SecureGenerator(KEY, nonce=5), SecureGenerator(KEY, nonce=5)
    for n in (16, 1000, 100_003):
        assert torch.equal(g_cpu.words(n), g_gpu.words(n, device="cuda").cpu())
    key = np.frombuffer(KEY, dtype="<u4")
    from opacus_b200.ops import _cuda

    out = torch.empty(16, dtype=torch.int32, device="cuda")
    _cuda.load().chacha_words(out, key.tolist(), 0x4A000000, 1 | (0x09000000 << 32))
    assert rfc7539_block_check((out.cpu().to(torch.int64) & 0xFFFFFFFF).tolist())
    # counters above 2^32 reach the kernel intact
    far = 1 << 40
    g_cpu.counter = g_gpu.counter = far
    assert torch.equal(g_cpu.words(64), g_gpu.words(64, device="cuda").cpu())


@pytest.mark.gpu
@pytest.mark.parametrize("draws", [1, 4])
@pytest.mark.parametrize("n", [1, 5, 4096, 1_000_003])
def test_cuda_gaussians_match_the_cpu_statement(draws, n):
    g_cpu, g_gpu = SecureGenerator(KEY), SecureGenerator(KEY)
    want = g_cpu.gaussian_like(torch.empty(n), 1.5, draws=draws)
    got = g_gpu.gaussian_like(torch.empty(n, device="cuda"), 1.5, draws=draws)
    assert g_cpu.counter == g_gpu.counter
    # same uniforms; log / sqrt / sincos differ by a few ulp between the two math libraries
    torch.testing.assert_close(got.cpu(), want, rtol=1e-4, atol=2e-5)
    if n > 100_000:
        assert abs(got.mean().item()) < 1e-2 and abs(got.std().item() - 1.5) < 1e-2


@pytest.mark.gpu
def test_secure_noise_on_cuda_parameters():
    from opacus_b200 import ops

    g = SecureGenerator(KEY)
    ref = torch.zeros(3, 1000, device="cuda", dtype=torch.bfloat16)
    z = ops.gaussian_like(ref, 2.0, generator=g, secure_mode=True)
    assert z.shape == ref.shape and z.dtype == torch.bfloat16 and z.is_cuda
    assert abs(z.float().std().item() - 2.0) < 0.1
    assert g.counter == 1 + (3000 * 4 + 15) // 16
