"""A cryptographically secure random generator for ``secure_mode``: ChaCha20 keystream, key from the OS entropy pool.

The reference gets its secure generator from the third-party ``torchcsprng`` package
(``opacus/privacy_engine.py:86-96``); when that package is not installed, ``PrivacyEngine(secure_mode=True)`` uses
:class:`SecureGenerator` instead.  The stream is the original ChaCha20 (20 rounds, 256-bit key, 64-bit block counter,
64-bit nonce); CUDA tensors are filled by a kernel that computes the same stream (``csrc/secure_rng.cu``), CPU tensors
by the vectorised numpy statement below, so a generator gives the same uniform words on both.

Numbers are derived from 32-bit keystream words ``w``:

* uniform on ``[0, 1)`` with 53 bits: ``((w0 >> 5) * 2^26 + (w1 >> 6)) / 2^53`` (sampling decisions),
* standard normal pairs by Box-Muller in fp32: ``u1 = (w0 + 1) / 2^32`` in ``(0, 1]``, ``u2 = w1 / 2^32``,
  ``r = sqrt(-2 ln u1)``, ``(r cos 2 pi u2, r sin 2 pi u2)``.

``gaussian_like(..., draws=4)`` is the rule of the reference's secure mode
(``opacus/optimizers/optimizer.py:143-160``): one draw is discarded, four independent draws are summed and halved, which
closes the gaps a single floating-point Gaussian leaves (Mironov, CCS 2012).
"""
from __future__ import annotations

import os
from typing import Optional, Sequence

import numpy as np
import torch

_CONSTANTS = np.frombuffer(b"expand 32-byte k", dtype="<u4")


def _rotl(x: np.ndarray, n: int) -> np.ndarray:
    return (x << np.uint32(n)) | (x >> np.uint32(32 - n))


def _quarter(s, a, b, c, d):
    s[a] += s[b]; s[d] ^= s[a]; s[d] = _rotl(s[d], 16)
    s[c] += s[d]; s[b] ^= s[c]; s[b] = _rotl(s[b], 12)
    s[a] += s[b]; s[d] ^= s[a]; s[d] = _rotl(s[d], 8)
    s[c] += s[d]; s[b] ^= s[c]; s[b] = _rotl(s[b], 7)


def chacha20_blocks(key: np.ndarray, nonce: int, first_block: int, n_blocks: int) -> np.ndarray:
    """``n_blocks`` 64-byte keystream blocks as ``uint32 [n_blocks, 16]`` (block ``first_block + i`` in row ``i``)."""
    counters = np.uint64(first_block) + np.arange(n_blocks, dtype=np.uint64)
    init = np.empty((16, n_blocks), dtype=np.uint32)
    init[0:4] = _CONSTANTS[:, None]
    init[4:12] = np.asarray(key, dtype=np.uint32)[:, None]
    init[12] = (counters & np.uint64(0xFFFFFFFF)).astype(np.uint32)
    init[13] = (counters >> np.uint64(32)).astype(np.uint32)
    init[14] = np.uint32(nonce & 0xFFFFFFFF)
    init[15] = np.uint32((nonce >> 32) & 0xFFFFFFFF)
    s = init.copy()
    with np.errstate(over="ignore"):
        for _ in range(10):
            _quarter(s, 0, 4, 8, 12); _quarter(s, 1, 5, 9, 13); _quarter(s, 2, 6, 10, 14); _quarter(s, 3, 7, 11, 15)
            _quarter(s, 0, 5, 10, 15); _quarter(s, 1, 6, 11, 12); _quarter(s, 2, 7, 8, 13); _quarter(s, 3, 4, 9, 14)
        s += init
    return np.ascontiguousarray(s.T)


def _normals_from_words(words: np.ndarray) -> np.ndarray:
    """Box-Muller on consecutive word pairs: ``[..., 2k]`` words -> ``[..., 2k]`` fp32 standard normals
    (pair ``j`` gives elements ``2j`` (cos) and ``2j + 1`` (sin))."""
    w = words.reshape(-1, 2)
    u1 = (w[:, 0].astype(np.float32) + np.float32(1.0)) * np.float32(2.0 ** -32)
    u2 = w[:, 1].astype(np.float32) * np.float32(2.0 ** -32)
    r = np.sqrt(np.float32(-2.0) * np.log(u1), dtype=np.float32)
    theta = np.float32(2.0 * np.pi) * u2
    out = np.empty_like(w, dtype=np.float32)
    out[:, 0] = r * np.cos(theta, dtype=np.float32)
    out[:, 1] = r * np.sin(theta, dtype=np.float32)
    return out.reshape(words.shape)


class SecureGenerator:
    """ChaCha20-based generator.  ``key``: 32 bytes (default: ``os.urandom(32)``); every call consumes whole 64-byte
    blocks and advances ``counter``, so no part of the stream is used twice."""

    def __init__(self, key: Optional[bytes] = None, nonce: int = 0):
        raw = os.urandom(32) if key is None else bytes(key)
        if len(raw) != 32:
            raise ValueError("SecureGenerator needs a 32-byte key")
        self.key = np.frombuffer(raw, dtype="<u4").copy()
        self.nonce = int(nonce) & 0xFFFFFFFFFFFFFFFF
        self.counter = 0

    # ---- stream bookkeeping
    def _take(self, n_blocks: int) -> int:
        first = self.counter
        self.counter += int(n_blocks)
        if self.counter >= 1 << 64:
            raise OverflowError("ChaCha20 block counter exhausted; create a new SecureGenerator")
        return first

    def get_state(self):
        return {"nonce": self.nonce, "counter": self.counter}

    def words(self, n: int, device="cpu") -> torch.Tensor:
        """``n`` keystream words as an int64 tensor of values in ``[0, 2^32)``."""
        blocks = (n + 15) // 16
        first = self._take(blocks)
        device = torch.device(device)
        if device.type == "cuda":
            from ..ops import _cuda

            out = torch.empty(blocks * 16, dtype=torch.int32, device=device)
            _cuda.load().chacha_words(out, self.key.tolist(), self.nonce, first)
            return (out[:n].to(torch.int64)) & 0xFFFFFFFF
        ks = chacha20_blocks(self.key, self.nonce, first, blocks).reshape(-1)[:n]
        return torch.from_numpy(ks.astype(np.int64))

    # ---- distributions
    def rand(self, n: int) -> torch.Tensor:
        """``n`` doubles uniform on ``[0, 1)`` (53 random bits each), on the CPU."""
        blocks = (2 * n + 15) // 16
        ks = chacha20_blocks(self.key, self.nonce, self._take(blocks), blocks).reshape(-1)[:2 * n].reshape(n, 2)
        hi = (ks[:, 0] >> np.uint32(5)).astype(np.float64)
        lo = (ks[:, 1] >> np.uint32(6)).astype(np.float64)
        return torch.from_numpy((hi * 67108864.0 + lo) / 9007199254740992.0)

    def randperm(self, n: int) -> torch.Tensor:
        """A uniformly random permutation of ``range(n)`` (sort of 53-bit keys; ties are broken by position and have
        probability about ``n^2 / 2^54``)."""
        return torch.argsort(self.rand(n), stable=True)

    def randint(self, high: int, n: int) -> torch.Tensor:
        return (self.rand(n) * high).floor().to(torch.int64).clamp_(max=high - 1)

    def gaussian_like(self, ref: torch.Tensor, std: float, draws: int = 1) -> torch.Tensor:
        """``N(0, std^2)`` with the shape, device and dtype of ``ref``.  ``draws=4``: the secure-mode rule (one block
        discarded, four draws summed and halved); element ``i`` uses words ``[4 i, 4 i + 4)`` of the call's stream.
        ``draws=1``: element ``i`` uses words ``[2 i, 2 i + 2)`` (the cosine branch)."""
        if draws not in (1, 4):
            raise ValueError("draws must be 1 or 4")
        n = ref.numel()
        if std == 0 or n == 0:
            return torch.zeros_like(ref)
        if draws == 4:
            self._take(1)                                  # the discarded draw
        per = 4 if draws == 4 else 2
        blocks = (n * per + 15) // 16
        first = self._take(blocks)
        if ref.is_cuda:
            from ..ops import _cuda

            out = torch.empty(n, dtype=torch.float32, device=ref.device)
            _cuda.load().chacha_normal(out, self.key.tolist(), self.nonce, first, float(std), draws)
        else:
            ks = chacha20_blocks(self.key, self.nonce, first, blocks).reshape(-1)[:n * per].reshape(n, per)
            z = _normals_from_words(ks)
            vals = z.sum(axis=1, dtype=np.float32) * np.float32(0.5) if draws == 4 else z[:, 0]
            out = torch.from_numpy(np.ascontiguousarray(vals * np.float32(std)))
        return out.reshape(ref.shape).to(ref.dtype)


class SecureRandomSampler(torch.utils.data.Sampler):
    """``RandomSampler`` whose permutation (or draws with replacement) come from a :class:`SecureGenerator`."""

    def __init__(self, data_source, generator: SecureGenerator, replacement: bool = False,
                 num_samples: Optional[int] = None):
        self.data_source = data_source
        self.generator = generator
        self.replacement = replacement
        self._num_samples = num_samples

    @property
    def num_samples(self) -> int:
        return len(self.data_source) if self._num_samples is None else self._num_samples

    def __iter__(self):
        n = len(self.data_source)
        if self.replacement:
            yield from self.generator.randint(n, self.num_samples).tolist()
            return
        left = self.num_samples
        while left > 0:
            perm = self.generator.randperm(n)[:left].tolist()
            yield from perm
            left -= len(perm)

    def __len__(self):
        return self.num_samples


def is_secure_generator(generator) -> bool:
    return isinstance(generator, SecureGenerator)


def rfc7539_block_check(words: Sequence[int]) -> bool:
    """True if ``words`` equals the keystream block of RFC 7539 section 2.3.2 (key 00..1f, counter 1, nonce
    00:00:00:09:00:00:00:4a:00:00:00:00); used by the tests of both implementations."""
    want = [0xe4e7f110, 0x15593bd1, 0x1fdd0f50, 0xc47120a3, 0xc7f4d1c7, 0x0368c033, 0x9aaa2204, 0x4e6cd4c3,
            0x466482d2, 0x09aa9f07, 0x05d7c214, 0xa2028bd9, 0xd19c12b5, 0xb94e16de, 0xe883d0cb, 0x4e3c50a2]
    return [int(w) & 0xFFFFFFFF for w in words] == want
