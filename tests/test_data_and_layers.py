"""Data loading, samplers, DP layers and validators on CPU."""
import pytest
import torch
import torch.nn as nn
from torch.utils.data import DataLoader, TensorDataset

from opacus_b200.data_loader import DPDataLoader, switch_generator, wrap_collate_with_empty
from opacus_b200.layers import DPGRU, DPLSTM, DPRNN, DPMultiheadAttention
from opacus_b200.utils.uniform_sampler import DistributedUniformWithReplacementSampler, UniformWithReplacementSampler


def test_poisson_sampler_statistics():
    g = torch.Generator().manual_seed(0)
    s = UniformWithReplacementSampler(num_samples=1000, sample_rate=0.1, generator=g, steps=200)
    sizes = [len(b) for b in s]
    assert len(sizes) == 200 and abs(sum(sizes) / 200 - 100) < 4
    assert len(UniformWithReplacementSampler(num_samples=10, sample_rate=0.25)) == 4


def test_distributed_sampler_partitions(monkeypatch):
    seen = []
    for rank in range(3):
        monkeypatch.setattr(torch.distributed, "get_world_size", lambda: 3)
        monkeypatch.setattr(torch.distributed, "get_rank", lambda r=rank: r)
        s = DistributedUniformWithReplacementSampler(total_size=100, sample_rate=1.0, steps=1,
                                                     generator=torch.Generator().manual_seed(rank))
        seen.append(torch.cat(list(s)))
    allidx = torch.cat(seen)
    assert sorted(allidx.tolist()) == list(range(100))
    s.set_epoch(1)
    assert not torch.equal(torch.cat(list(s)).sort().values, seen[2].sort().values)


def test_dp_data_loader_and_empty_batches():
    ds = TensorDataset(torch.randn(50, 3), torch.randint(0, 2, (50,)))
    dl = DPDataLoader.from_data_loader(DataLoader(ds, batch_size=10), generator=torch.Generator().manual_seed(1))
    assert dl.sample_rate == pytest.approx(0.2) and len(dl) == 5
    assert all(x.shape[1] == 3 for x, _ in dl)
    tiny = DPDataLoader(ds, sample_rate=1e-6, generator=torch.Generator().manual_seed(1))
    x, y = next(iter(tiny))
    assert x.shape == (0, 3) and y.shape == (0,) and y.dtype == torch.int64
    coll = wrap_collate_with_empty(collate_fn=torch.utils.data.default_collate, rand_on_empty=True)
    coll([(torch.zeros(3), 1), (torch.zeros(3), 0)])
    x, y = coll([])
    assert x.shape == (1, 3)
    with pytest.raises(ValueError):
        class It(torch.utils.data.IterableDataset):
            def __iter__(self):
                yield 1

        DPDataLoader.from_data_loader(DataLoader(It()))


def test_switch_generator():
    ds = TensorDataset(torch.arange(20).float())
    g1, g2 = torch.Generator().manual_seed(5), torch.Generator().manual_seed(5)
    a = [b[0].tolist() for b in switch_generator(data_loader=DataLoader(ds, batch_size=4, shuffle=True), generator=g1)]
    b = [b[0].tolist() for b in switch_generator(data_loader=DataLoader(ds, batch_size=4, shuffle=True), generator=g2)]
    assert a == b


@pytest.mark.parametrize("dp,ref", [(DPLSTM, nn.LSTM), (DPGRU, nn.GRU), (DPRNN, nn.RNN)])
def test_dp_rnn_matches_torch(dp, ref):
    torch.manual_seed(0)
    a, b = dp(4, 6, num_layers=2, bidirectional=True, batch_first=True), ref(4, 6, num_layers=2, bidirectional=True, batch_first=True)
    assert set(a.state_dict()) == set(b.state_dict())
    a.load_state_dict(b.state_dict())
    x = torch.randn(3, 5, 4, requires_grad=True)
    ya, _ = a(x)
    yb, _ = b(x)
    assert torch.allclose(ya, yb, atol=1e-5)
    ga, = torch.autograd.grad(ya.sum(), x)
    gb, = torch.autograd.grad(yb.sum(), x)
    assert torch.allclose(ga, gb, atol=1e-5)


def test_dp_mha_matches_torch():
    torch.manual_seed(0)
    a, b = DPMultiheadAttention(8, 2, batch_first=True), nn.MultiheadAttention(8, 2, batch_first=True)
    a.load_state_dict(b.state_dict())
    b.load_state_dict(a.state_dict())
    x = torch.randn(2, 5, 8)
    for need in (True, False):
        ya, wa = a(x, x, x, need_weights=need)
        yb, wb = b(x, x, x, need_weights=need)
        assert torch.allclose(ya, yb, atol=1e-5)


def test_fused_cross_entropy_cpu_fallback():
    from opacus_b200.layers import FusedCrossEntropyLoss

    torch.manual_seed(0)
    logits = torch.randn(6, 11, requires_grad=True)
    target = torch.tensor([1, 2, -100, 4, 0, 10])
    for red in ("none", "mean", "sum"):
        got = FusedCrossEntropyLoss(reduction=red)(logits, target)
        want = torch.nn.functional.cross_entropy(logits, target, reduction=red)
        torch.testing.assert_close(got, want)


def test_distributed_sampler_with_explicit_replicas():
    """Tensor-parallel ranks of one group pass the same (replicas, rank, generator state) and draw the same batches;
    different groups draw from disjoint slices of the data."""
    import torch
    from opacus_b200.utils.uniform_sampler import DistributedUniformWithReplacementSampler as Sampler

    def draw(rank, seed):
        s = Sampler(total_size=200, sample_rate=0.1, num_replicas=2, rank=rank, generator=torch.Generator().manual_seed(seed))
        return [list(map(int, b)) for b in s]

    assert draw(0, 5) == draw(0, 5)
    a, b = draw(0, 5), draw(1, 6)
    assert not ({i for x in a for i in x} & {i for x in b for i in x})
    with pytest.raises(ValueError):
        Sampler(total_size=10, sample_rate=0.5, num_replicas=2, rank=2)
