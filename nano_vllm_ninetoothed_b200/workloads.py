"""Seeded synthetic inputs of the benchmark shapes, plus their algorithmic byte/flop counts.

Values are drawn with a `torch.Generator` so that the CPU checker and the CUDA kernels see
identical bits: small cases are generated on the CPU in fp32, cast, and copied; the large
decode pool is generated directly on the device with a seeded CUDA generator.

Shapes follow how nano-vLLM builds its inputs (nanovllm/engine/model_runner.py:120-180):
int32 `block_tables` padded with -1, int32 `context_lens` that include the token being
decoded, int32 `slot_mapping`, int32 `cu_seqlens`, int64 token ids.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

PAGE = 256       # nano-vLLM's KV block size (nanovllm/engine/sequence.py:15)
HEAD_DIM = 128


def _gen(seed: int, device="cpu") -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def _randn(shape, g: torch.Generator, dtype, std=1.0, mean=0.0) -> torch.Tensor:
    """fp32 draw on the CPU generator, scaled, then rounded to `dtype`."""
    x = torch.randn(shape, generator=g, dtype=torch.float32)
    if std != 1.0:
        x = x * std
    if mean != 0.0:
        x = x + mean
    return x.to(dtype)


# --------------------------------------------------------------------------- paged decode
@dataclass
class DecodeCase:
    q: torch.Tensor               # [B, 1, Hq, d]
    k_cache: torch.Tensor         # [NB, page, Hkv, d]
    v_cache: torch.Tensor
    cache_seqlens: torch.Tensor   # int32 [B]
    block_table: torch.Tensor     # int32 [B, max_blocks], -1 padded
    softmax_scale: float
    hq: int
    hkv: int
    page: int
    meta: dict = field(default_factory=dict)

    def to(self, device) -> "DecodeCase":
        return DecodeCase(self.q.to(device), self.k_cache.to(device), self.v_cache.to(device),
                          self.cache_seqlens.to(device), self.block_table.to(device),
                          self.softmax_scale, self.hq, self.hkv, self.page, dict(self.meta))

    def algorithmic_bytes(self) -> int:
        return decode_bytes(self.cache_seqlens, self.hq, self.hkv, self.q.shape[-1], self.page,
                            self.q.element_size())

    def flops(self) -> int:
        return 4 * self.hq * self.q.shape[-1] * int(self.cache_seqlens.sum().item())


def decode_bytes(lens: torch.Tensor, hq: int, hkv: int, d: int, page: int, esize: int = 2) -> int:
    """K and V of every live token once, q and o once, lens, and the live table entries."""
    lens = lens.to(torch.int64).cpu()
    batch = lens.numel()
    kv = int(lens.sum().item()) * hkv * d * 2 * esize
    qo = 2 * batch * hq * d * esize
    idx = 4 * batch + 4 * int(((lens + page - 1) // page).sum().item())
    return kv + qo + idx


def make_decode_case(seed: int = 0, batch: int = 8, len_lo: int = 128, len_hi: int = 1024,
                     hq: int = 16, hkv: int = 8, head_dim: int = HEAD_DIM, page: int = PAGE,
                     num_blocks: int | None = None, dtype=torch.bfloat16, device="cpu",
                     lens: list[int] | None = None, poison: bool = False,
                     cache_on_device: bool = False, spare_blocks: int = 4) -> DecodeCase:
    """Paged decode inputs.  Each block-table row is the next `ceil(len/page)` ids of a seeded
    permutation of the physical blocks.  With `poison`, every slot that no live token occupies
    (dead tail of the last page, unused pages) is NaN, so reading one shows up in the output.
    `cache_on_device` draws the KV pool with a CUDA generator instead (for multi-GB pools)."""
    g = _gen(seed)
    if lens is None:
        lens_t = torch.randint(len_lo, len_hi + 1, (batch,), generator=g, dtype=torch.int64)
    else:
        lens_t = torch.tensor(lens, dtype=torch.int64)
        batch = lens_t.numel()
    blocks_per_seq = (lens_t + page - 1) // page
    need = int(blocks_per_seq.sum().item())
    if num_blocks is None:
        num_blocks = need + spare_blocks
    if num_blocks < need:
        raise ValueError(f"{need} blocks needed, pool has {num_blocks}")
    perm = torch.randperm(num_blocks, generator=g)
    max_blocks = max(1, int(blocks_per_seq.max().item()))
    table = torch.full((batch, max_blocks), -1, dtype=torch.int32)
    cursor = 0
    for b in range(batch):
        n = int(blocks_per_seq[b])
        table[b, :n] = perm[cursor:cursor + n].to(torch.int32)
        cursor += n
    q = _randn((batch, 1, hq, head_dim), g, dtype)
    shape = (num_blocks, page, hkv, head_dim)
    if cache_on_device:
        gd = _gen(seed + 1, device)
        k_cache = torch.randn(shape, generator=gd, device=device, dtype=dtype)
        v_cache = torch.randn(shape, generator=gd, device=device, dtype=dtype)
    else:
        k_cache = _randn(shape, g, dtype)
        v_cache = _randn(shape, g, dtype)
    case = DecodeCase(q, k_cache, v_cache, lens_t.to(torch.int32), table,
                      1.0 / math.sqrt(head_dim), hq, hkv, page,
                      {"seed": seed, "num_blocks": num_blocks})
    if poison:
        live = torch.zeros(num_blocks, page, dtype=torch.bool)
        for b in range(batch):
            ln = int(lens_t[b])
            for i in range(int(blocks_per_seq[b])):
                live[int(table[b, i]), : min(page, ln - i * page)] = True
        dead = ~live.to(k_cache.device)
        case.k_cache[dead] = float("nan")
        case.v_cache[dead] = float("nan")
    if not cache_on_device and str(device) != "cpu":
        case = case.to(device)
    elif cache_on_device:
        case.q = case.q.to(device)
        case.cache_seqlens = case.cache_seqlens.to(device)
        case.block_table = case.block_table.to(device)
    return case


# --------------------------------------------------------------------------- varlen prefill
@dataclass
class PrefillCase:
    q: torch.Tensor               # [T, Hq, d]
    k: torch.Tensor               # [T, Hkv, d]
    v: torch.Tensor               # [T, Hkv, d] (a strided view when `strided_v`)
    cu_seqlens: torch.Tensor      # int32 [B + 1]
    max_seqlen: int
    softmax_scale: float
    hq: int
    hkv: int
    lens: list[int] = field(default_factory=list)

    def to(self, device) -> "PrefillCase":
        return PrefillCase(self.q.to(device), self.k.to(device), self.v.to(device),
                           self.cu_seqlens.to(device), self.max_seqlen, self.softmax_scale,
                           self.hq, self.hkv, list(self.lens))

    def flops(self) -> int:
        return prefill_flops(self.lens, self.hq, self.q.shape[-1])

    def algorithmic_bytes(self) -> int:
        t, d, es = self.q.shape[0], self.q.shape[-1], self.q.element_size()
        return 2 * t * self.hq * d * es + 2 * t * self.hkv * d * es


def prefill_flops(lens, hq: int, d: int) -> int:
    """Causal pairs only: QK^T and PV at 2*d flops per (query, key) pair each."""
    return 4 * d * hq * sum(n * (n + 1) // 2 for n in lens)


def make_prefill_case(seed: int = 0, batch: int = 8, len_lo: int = 64, len_hi: int = 2048,
                      hq: int = 16, hkv: int = 8, head_dim: int = HEAD_DIM,
                      dtype=torch.bfloat16, device="cpu", lens: list[int] | None = None,
                      strided_v: bool = False) -> PrefillCase:
    """Packed varlen prefill inputs.  With `strided_v`, q/k/v are the three column slices of
    one `[T, (Hq+2Hkv)*d]` activation, as the qkv projection produces them
    (nanovllm/models/qwen3.py:74-78)."""
    g = _gen(seed)
    if lens is None:
        lens = torch.randint(len_lo, len_hi + 1, (batch,), generator=g).tolist()
    total = sum(lens)
    cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(torch.tensor(lens, dtype=torch.int64), 0).to(torch.int32)
    if strided_v:
        qkv = _randn((total, (hq + 2 * hkv) * head_dim), g, dtype).to(device)
        qs, ks = hq * head_dim, hkv * head_dim
        q = qkv[:, :qs].view(total, hq, head_dim)
        k = qkv[:, qs:qs + ks].view(total, hkv, head_dim)
        v = qkv[:, qs + ks:].view(total, hkv, head_dim)
    else:
        q = _randn((total, hq, head_dim), g, dtype).to(device)
        k = _randn((total, hkv, head_dim), g, dtype).to(device)
        v = _randn((total, hkv, head_dim), g, dtype).to(device)
    return PrefillCase(q, k, v, cu.to(device), max(lens) if lens else 0,
                       1.0 / math.sqrt(head_dim), hq, hkv, list(lens))


# --------------------------------------------------------------------------- bandwidth ops
def make_store_case(seed: int = 0, n_tokens: int = 4096, hkv: int = 8, head_dim: int = HEAD_DIM,
                    num_blocks: int = 128, page: int = PAGE, dtype=torch.bfloat16, device="cpu",
                    strided: bool = True, skip_every: int = 0):
    """(key, value, k_cache, v_cache, slot_mapping): non-colliding random slots into zeroed
    caches; with `strided`, key/value are column slices of a wider activation; with
    `skip_every` > 0 every n-th slot is -1 (padding of a replayed decode graph)."""
    g = _gen(seed)
    d = hkv * head_dim
    if strided:
        buf = _randn((n_tokens, 4 * d), g, dtype).to(device)
        key = buf[:, d:2 * d].view(n_tokens, hkv, head_dim)
        value = buf[:, 2 * d:3 * d].view(n_tokens, hkv, head_dim)
    else:
        key = _randn((n_tokens, hkv, head_dim), g, dtype).to(device)
        value = _randn((n_tokens, hkv, head_dim), g, dtype).to(device)
    slots = torch.randperm(num_blocks * page, generator=g)[:n_tokens].to(torch.int32)
    if skip_every:
        slots[::skip_every] = -1
    k_cache = torch.zeros((num_blocks, page, hkv, head_dim), dtype=dtype, device=device)
    v_cache = torch.zeros_like(k_cache)
    return key, value, k_cache, v_cache, slots.to(device)


def store_bytes(n_tokens: int, hkv: int, d: int, esize: int = 2) -> int:
    return n_tokens * (2 * hkv * d * esize + 2 * hkv * d * esize + 4)


def make_rms_case(seed: int = 0, rows: int = 4096, hidden: int = 1024, dtype=torch.bfloat16,
                  device="cpu"):
    """(x, residual, weight): N(0,1) activations, weight ~ N(1, 0.02)."""
    g = _gen(seed)
    x = _randn((rows, hidden), g, dtype).to(device)
    r = _randn((rows, hidden), g, dtype).to(device)
    w = _randn((hidden,), g, dtype, std=0.02, mean=1.0).to(device)
    return x, r, w


def add_rms_bytes(rows: int, hidden: int, esize: int = 2) -> int:
    return rows * hidden * esize * 4 + hidden * esize


def make_embedding_case(seed: int = 0, n_ids: int = 4096, vocab: int = 151936, hidden: int = 1024,
                        dtype=torch.bfloat16, device="cpu"):
    """(ids int64, table ~ N(0, 0.02)); the first two ids are forced to 0 and vocab-1."""
    g = _gen(seed)
    ids = torch.randint(0, vocab, (n_ids,), generator=g, dtype=torch.int64)
    if n_ids >= 2:
        ids[0], ids[1] = 0, vocab - 1
    if str(device) != "cpu":
        gd = _gen(seed + 1, device)
        table = (torch.randn((vocab, hidden), generator=gd, device=device, dtype=torch.float32) * 0.02).to(dtype)
    else:
        table = _randn((vocab, hidden), g, dtype, std=0.02)
    return ids.to(device), table


def embedding_bytes(n_ids: int, hidden: int, esize: int = 2) -> int:
    return n_ids * (2 * hidden * esize + 8)


# --------------------------------------------------------------------------- named configs
def config_lens(name: str, seed: int = 0) -> list[int]:
    """Sequence lengths of the named benchmark configurations."""
    g = _gen(seed)
    spec = {
        "decode_small": (8, 128, 1024),       # Qwen3-0.6B heads, 8 sequences
        "prefill_small": (8, 64, 2048),       # Qwen3-0.6B heads, 8 sequences
        "prefill_8b": (16, 256, 4096),        # Qwen3-8B heads, 16 sequences
        "decode_8b": (256, 512, 8192),        # Qwen3-8B heads, 256 sequences
    }[name]
    return torch.randint(spec[1], spec[2] + 1, (spec[0],), generator=g).tolist()


# --------------------------------------------------------------------------- KV-head sharding
def kv_head_range(hkv: int, rank: int, world: int) -> tuple[int, int]:
    """KV heads owned by `rank` under nano-vLLM's tensor parallelism: contiguous groups of
    `hkv // world` heads (nanovllm/models/qwen3.py:29-38); query heads follow as G * range."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} for world size {world}")
    if hkv % world != 0:
        raise ValueError(f"{hkv} KV heads do not split over {world} ranks")
    per = hkv // world
    return rank * per, (rank + 1) * per


def shard_decode_case(case: DecodeCase, rank: int, world: int) -> DecodeCase:
    """This rank's slice of a decode case: its KV heads of both caches and the matching query
    heads; lengths and block tables are replicated, exactly as the engine broadcasts them."""
    lo, hi = kv_head_range(case.hkv, rank, world)
    g = case.hq // case.hkv
    return DecodeCase(case.q[:, :, lo * g:hi * g].contiguous(),
                      case.k_cache[:, :, lo:hi].contiguous(), case.v_cache[:, :, lo:hi].contiguous(),
                      case.cache_seqlens, case.block_table, case.softmax_scale,
                      (hi - lo) * g, hi - lo, case.page, dict(case.meta, rank=rank, world=world))


def shard_prefill_case(case: PrefillCase, rank: int, world: int) -> PrefillCase:
    lo, hi = kv_head_range(case.hkv, rank, world)
    g = case.hq // case.hkv
    return PrefillCase(case.q[:, lo * g:hi * g].contiguous(), case.k[:, lo:hi].contiguous(),
                       case.v[:, lo:hi].contiguous(), case.cu_seqlens, case.max_seqlen,
                       case.softmax_scale, (hi - lo) * g, hi - lo, list(case.lens))
