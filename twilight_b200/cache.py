"""Paged KV cache in the HBM layout the kernels read, and the INT4 slab format.

Layout (page size 16, head_dim 128, quantisation group 32):

* ``k_pages`` / ``v_pages``  ``[num_pages, H_kv, 16, 128]``   fp16 or bf16 (4 KiB per page and head)
* ``k4_pages``               ``[num_pages, H_kv, 1280]`` uint8: 1024 code bytes (token-major, byte j
  of a token = channel 2j in the low nibble, 2j+1 in the high nibble) then 16 x 4 x {fp16 scale,
  fp16 minimum}; a token costs 80 bytes.  ``value = code*scale + minimum``.
* ``kmeta``                  ``[num_pages, H_kv, 2, 128]`` channel-wise {min, max} of the page
* page table                 FlashInfer-style CSR (``kv_indptr``, ``kv_indices``, ``kv_last_page_len``),
  the one the reference's GEMV benchmark builds (benchmark/efficiency/bench_gemv.py:437-443).

The pack/unpack helpers below only move bits (they define the format and serve the tests); the
quantiser itself is the CUDA kernel behind ``twilight_b200.kernel.quantize_k_pages``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

PAGE = 16
HEAD_DIM = 128
GROUP = 32
K4_SLAB_BYTES = 1280


def pack_k4(codes: torch.Tensor, scale: torch.Tensor, zmin: torch.Tensor) -> torch.Tensor:
    """codes ``[...,16,128]`` uint8 (0..15), scale/zmin ``[...,16,4]`` -> slabs ``[...,1280]`` uint8."""
    lead = codes.shape[:-2]
    c = codes.to(torch.uint8).reshape(*lead, PAGE, HEAD_DIM // 2, 2)
    packed = (c[..., 0] | (c[..., 1] << 4)).reshape(*lead, PAGE * HEAD_DIM // 2)
    sz = torch.stack([scale.to(torch.float16), zmin.to(torch.float16)], dim=-1)  # [...,16,4,2]
    sz_bytes = sz.contiguous().view(torch.uint8).reshape(*lead, PAGE * 4 * 4)
    return torch.cat([packed, sz_bytes], dim=-1).contiguous()


def unpack_k4(slab: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Inverse of :func:`pack_k4`: returns ``(codes [...,16,128] uint8, scale, zmin [...,16,4] fp16)``."""
    lead = slab.shape[:-1]
    packed = slab[..., : PAGE * HEAD_DIM // 2].reshape(*lead, PAGE, HEAD_DIM // 2)
    codes = torch.stack([packed & 0xF, packed >> 4], dim=-1).reshape(*lead, PAGE, HEAD_DIM)
    sz = slab[..., PAGE * HEAD_DIM // 2:].contiguous().view(torch.float16).reshape(*lead, PAGE, 4, 2)
    return codes, sz[..., 0], sz[..., 1]


def quest_max_k(token_budget: int, max_pages: int) -> int:
    """Pages Quest keeps for a token budget (twilight/pyimpl/quest.py:93-98)."""
    k = max(1, token_budget // PAGE) + (1 if token_budget % PAGE else 0)
    return min(k, max_pages)


@dataclass
class PagedKVCache:
    """Device tensors of one attention layer's cache plus its page table."""
    k_pages: torch.Tensor
    v_pages: torch.Tensor
    k4_pages: Optional[torch.Tensor]
    kmeta: Optional[torch.Tensor]
    kv_indptr: torch.Tensor          # int32 [B+1]
    kv_indices: torch.Tensor         # int32 [sum pages]
    kv_last_page_len: torch.Tensor   # int32 [B]
    seq_lens: List[int]              # host copy of the token counts
    capacity_pages: Optional[int] = None   # pages per sequence a growing cache reserves (sizes workspaces)

    @property
    def batch(self) -> int:
        return len(self.seq_lens)

    @property
    def num_kv_heads(self) -> int:
        return self.k_pages.shape[1]

    @property
    def max_pages(self) -> int:
        return max((l + PAGE - 1) // PAGE for l in self.seq_lens)

    @property
    def dtype(self) -> torch.dtype:
        return self.k_pages.dtype

    @property
    def device(self) -> torch.device:
        return self.k_pages.device

    # ---- construction -------------------------------------------------------------------------
    @staticmethod
    def page_table(seq_lens: Sequence[int], device, shuffle_seed: Optional[int] = None
                   ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, int]:
        """CSR page table for the given token counts; physical page ids are consecutive, or a
        seeded random permutation when ``shuffle_seed`` is given."""
        n_pages = [(l + PAGE - 1) // PAGE for l in seq_lens]
        total = sum(n_pages)
        indptr = torch.zeros(len(seq_lens) + 1, dtype=torch.int32)
        indptr[1:] = torch.tensor(n_pages, dtype=torch.int32).cumsum(0)
        if shuffle_seed is None:
            indices = torch.arange(total, dtype=torch.int32)
        else:
            g = torch.Generator().manual_seed(shuffle_seed)
            indices = torch.randperm(total, generator=g).to(torch.int32)
        last = torch.tensor([(l - 1) % PAGE + 1 for l in seq_lens], dtype=torch.int32)
        return indptr.to(device), indices.to(device), last.to(device), total

    @classmethod
    def from_dense(cls, k: torch.Tensor, v: torch.Tensor, seq_lens: Optional[Sequence[int]] = None,
                   shuffle_seed: Optional[int] = None, build_aux: bool = True) -> "PagedKVCache":
        """k, v ``[B,H_kv,L,128]`` (per KV head, not expanded) -> paged cache on k's device.
        With ``build_aux`` the INT4 slabs and the page metadata are produced by the CUDA kernels."""
        b, hkv, l, d = k.shape
        assert d == HEAD_DIM
        seq_lens = [l] * b if seq_lens is None else list(seq_lens)
        indptr, indices, last, total = cls.page_table(seq_lens, k.device, shuffle_seed)
        k_pages = torch.zeros(total, hkv, PAGE, d, dtype=k.dtype, device=k.device)
        v_pages = torch.zeros_like(k_pages)
        idx_host = indices.cpu()
        ptr_host = indptr.cpu()
        for i, n in enumerate(seq_lens):
            npg = (n + PAGE - 1) // PAGE
            pad = npg * PAGE - n
            phys = idx_host[ptr_host[i]: ptr_host[i + 1]].long().to(k.device)
            for src, dst in ((k, k_pages), (v, v_pages)):
                x = src[i, :, :n]
                if pad:
                    x = torch.cat([x, torch.zeros(hkv, pad, d, dtype=x.dtype, device=x.device)], 1)
                dst[phys] = x.reshape(hkv, npg, PAGE, d).permute(1, 0, 2, 3)
        cache = cls(k_pages, v_pages, None, None, indptr, indices, last, seq_lens)
        if build_aux:
            cache.build_aux()
        return cache

    def build_aux(self) -> None:
        """(Re)builds INT4 slabs and page metadata from ``k_pages`` with the CUDA kernels."""
        from .kernel import ops
        self.k4_pages = ops.quantize_k_pages(self.k_pages, self.k4_pages)
        self.kmeta = ops.build_page_meta(self.k_pages, self.kv_indptr, self.kv_indices,
                                         self.kv_last_page_len, max_pages=self.max_pages,
                                         kmeta=self.kmeta)

    # ---- inspection (tests, baselines) ------------------------------------------------------------
    def _phys(self, b: int) -> torch.Tensor:
        lo, hi = int(self.kv_indptr[b]), int(self.kv_indptr[b + 1])
        return self.kv_indices[lo:hi].long()

    def dense_kv(self, b: int, kvh: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """K, V ``[L_b,128]`` of one sequence and KV head, gathered through the page table."""
        phys, n = self._phys(b), self.seq_lens[b]
        k = self.k_pages[phys, kvh].reshape(-1, HEAD_DIM)[:n]
        v = self.v_pages[phys, kvh].reshape(-1, HEAD_DIM)[:n]
        return k, v

    def dense_k4(self, b: int, kvh: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """INT4 ``(codes [L_b,128], scale [L_b,4], zmin [L_b,4])`` of one sequence and KV head."""
        phys, n = self._phys(b), self.seq_lens[b]
        codes, scale, zmin = unpack_k4(self.k4_pages[phys, kvh])
        return (codes.reshape(-1, HEAD_DIM)[:n], scale.reshape(-1, 4)[:n], zmin.reshape(-1, 4)[:n])

    def dense_meta(self, b: int, kvh: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """Page metadata ``(kmin, kmax) [n_pages_b,128]`` of one sequence and KV head."""
        phys = self._phys(b)
        m = self.kmeta[phys, kvh]
        return m[:, 0], m[:, 1]


class GrowingPagedCache:
    """A paged cache of one attention layer that grows by one token per sequence and step.

    Every sequence owns ``ceil(max_len / 16)`` consecutive physical pages from the start, so growing
    never moves data: only the page table (a few integers, rebuilt on the host) changes.  All
    sequences have the same length, as in a batch without padding.  ``view`` is the
    :class:`PagedKVCache` the kernels read."""

    def __init__(self, batch: int, num_kv_heads: int, max_len: int, dtype: torch.dtype, device) -> None:
        self.batch, self.max_len = batch, max_len
        self.pages_per_seq = (max_len + PAGE - 1) // PAGE
        total = batch * self.pages_per_seq
        self.k_pages = torch.zeros(total, num_kv_heads, PAGE, HEAD_DIM, dtype=dtype, device=device)
        self.v_pages = torch.zeros_like(self.k_pages)
        self.k4_pages = torch.zeros(total, num_kv_heads, K4_SLAB_BYTES, dtype=torch.uint8, device=device)
        self.kmeta = torch.zeros(total, num_kv_heads, 2, HEAD_DIM, dtype=dtype, device=device)
        self.length = 0
        self.view: Optional[PagedKVCache] = None

    def _set_length(self, n: int) -> None:
        if n > self.max_len:
            raise ValueError(f"cache holds {self.max_len} tokens per sequence, asked for {n}")
        dev = self.k_pages.device
        npg = (n + PAGE - 1) // PAGE
        if self.view is None or (self.length + PAGE - 1) // PAGE != npg:
            first = torch.arange(self.batch, dtype=torch.int32)[:, None] * self.pages_per_seq
            indices = (first + torch.arange(npg, dtype=torch.int32)[None, :]).reshape(-1).to(dev)
            indptr = (torch.arange(self.batch + 1, dtype=torch.int32) * npg).to(dev)
        else:
            indptr, indices = self.view.kv_indptr, self.view.kv_indices
        last = torch.full((self.batch,), (n - 1) % PAGE + 1, dtype=torch.int32, device=dev)
        self.view = PagedKVCache(self.k_pages, self.v_pages, self.k4_pages, self.kmeta, indptr, indices, last,
                                 [n] * self.batch, capacity_pages=self.pages_per_seq)
        self.length = n

    def load(self, k: torch.Tensor, v: torch.Tensor) -> None:
        """Replaces the contents with ``k, v [B,H_kv,L,128]`` (a prefill) and builds the INT4 slabs
        and the page metadata with the CUDA kernels."""
        b, hkv, n, d = k.shape
        assert b == self.batch and d == HEAD_DIM and n >= 1
        self._set_length(n)
        npg = (n + PAGE - 1) // PAGE
        pad = npg * PAGE - n
        for src, dst in ((k, self.k_pages), (v, self.v_pages)):
            x = src.to(dst.dtype)
            if pad:
                x = torch.cat([x, torch.zeros(b, hkv, pad, d, dtype=x.dtype, device=x.device)], 2)
            pages = dst.view(b, self.pages_per_seq, hkv, PAGE, d)
            pages[:, :npg] = x.reshape(b, hkv, npg, PAGE, d).permute(0, 2, 1, 3, 4)
        self.view.build_aux()

    def append(self, new_k: torch.Tensor, new_v: torch.Tensor) -> None:
        """Adds one token per sequence (``new_k, new_v [B,H_kv,128]``): K/V rows, INT4 codes and the
        page's metadata, by the append kernel."""
        from .kernel import ops
        self._set_length(self.length + 1)
        c = self.view
        ops.append_kv(new_k.to(self.k_pages.dtype).contiguous(), new_v.to(self.k_pages.dtype).contiguous(),
                      c.k_pages, c.v_pages, c.k4_pages, c.kmeta, c.kv_indptr, c.kv_indices, c.kv_last_page_len)
