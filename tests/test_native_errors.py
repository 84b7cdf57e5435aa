"""How the native module reports a kernel that gave up on a bounded wait (host part; no GPU needed)."""
import pytest


def test_wait_timeout_becomes_comm_timeout_error():
    try:
        from opacus_b200 import _C  # noqa: F401
    except ImportError:
        pytest.skip("native extension not built")
    from opacus_b200.ops import _cuda
    from opacus_b200.utils.errors import CommTimeoutError

    native = _cuda.load()
    with pytest.raises(CommTimeoutError, match="bounded wait"):
        native._raise_wait_timeout_for_test()
    assert issubclass(CommTimeoutError, RuntimeError)
    # other errors pass through unchanged
    import torch

    with pytest.raises(RuntimeError) as info:
        native.scale_rows(torch.zeros(2, 8), None, 1, 1.0)          # CPU tensor: rejected by the binding
    assert not isinstance(info.value, CommTimeoutError)
