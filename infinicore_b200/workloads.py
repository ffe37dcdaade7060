"""Seeded synthetic decode workloads: the five benchmark configurations plus a free-form
builder for test cases.

The reference measures on no external dataset; its tests draw random tensors
(test/infiniop/paged_attention.py:150-173).  These generators produce the shapes, sizes and
value distributions of the benchmark configurations from a seed, on CPU (so a CPU checker and
the GPU see identical bits) or directly on a GPU for the large ones.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch


@dataclass
class DecodeCase:
    name: str
    dtype: torch.dtype
    num_heads: int
    num_kv_heads: int
    head_size: int
    block_size: int
    scale: float
    q: torch.Tensor              # [num_seqs, num_heads, head_size]
    k_cache: torch.Tensor        # [num_blocks, num_kv_heads, block_size, head_size]
    v_cache: torch.Tensor
    block_tables: torch.Tensor   # [num_seqs, max_blocks_per_seq] int64
    seq_lens: torch.Tensor       # [num_seqs] int64
    new_k: torch.Tensor          # [num_seqs, num_kv_heads, head_size] rows for the newest token
    new_v: torch.Tensor
    slot_mapping: torch.Tensor   # [num_seqs] int64: slot of token seq_len - 1
    extra: dict = field(default_factory=dict)

    @property
    def num_seqs(self) -> int:
        return self.q.shape[0]

    @property
    def total_tokens(self) -> int:
        return int(self.seq_lens.clamp(min=0).sum().item())

    @property
    def kv_bytes(self) -> int:
        """Algorithmic bytes of one attention pass: every K and V element of every live token once."""
        elem = self.k_cache.element_size()
        return self.total_tokens * self.num_kv_heads * (self.head_size + self.v_cache.shape[3]) * elem

    @property
    def caching_bytes(self) -> int:
        elem = self.k_cache.element_size()
        return 2 * self.num_seqs * self.num_kv_heads * (self.head_size + self.v_cache.shape[3]) * elem

    def to(self, device) -> "DecodeCase":
        moved = {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in self.__dict__.items()}
        return DecodeCase(**moved)


def _randn(shape, dtype, std, gen, device, chunk_elems=1 << 28):
    """N(0, std) in `dtype`, drawn in chunks so a multi-GB pool never needs an fp32 twin."""
    out = torch.empty(shape, dtype=dtype, device=device)
    flat = out.view(-1)
    for start in range(0, flat.numel(), chunk_elems):
        n = min(chunk_elems, flat.numel() - start)
        flat[start:start + n] = (torch.randn(n, generator=gen, device=device, dtype=torch.float32) * std).to(dtype)
    return out


def build_case(name, *, dtype, seq_lens, num_heads, num_kv_heads, head_size, block_size, num_blocks=None,
               max_blocks_per_seq=None, std=1.0, seed=0, device="cpu", shuffle_tables=True, value_size=None,
               slack_blocks=0) -> DecodeCase:
    """Builds one decode problem.  Block tables take distinct pool blocks in (seeded) random order;
    table entries past a sequence's last block are 0 and must never be read."""
    device = torch.device(device)
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    cpu_gen = torch.Generator()
    cpu_gen.manual_seed(seed + 1)

    seq_lens = torch.as_tensor(seq_lens, dtype=torch.int64)
    num_seqs = seq_lens.numel()
    blocks_per_seq = (seq_lens.clamp(min=0) + block_size - 1) // block_size
    need = int(blocks_per_seq.sum().item())
    if num_blocks is None:
        num_blocks = max(1, need + slack_blocks)
    assert need <= num_blocks, "pool too small for these sequence lengths"
    if max_blocks_per_seq is None:
        max_blocks_per_seq = max(1, int(blocks_per_seq.max().item()))
    value_size = value_size or head_size

    order = torch.randperm(num_blocks, generator=cpu_gen) if shuffle_tables else torch.arange(num_blocks)
    block_tables = torch.zeros((num_seqs, max_blocks_per_seq), dtype=torch.int64)
    slot_mapping = torch.full((num_seqs,), -1, dtype=torch.int64)
    cursor = 0
    for i in range(num_seqs):
        n = int(blocks_per_seq[i])
        block_tables[i, :n] = order[cursor:cursor + n]
        cursor += n
        ln = int(seq_lens[i])
        if ln > 0:
            slot_mapping[i] = block_tables[i, (ln - 1) // block_size] * block_size + (ln - 1) % block_size

    q = _randn((num_seqs, num_heads, head_size), dtype, std, gen, device)
    k_cache = _randn((num_blocks, num_kv_heads, block_size, head_size), dtype, std, gen, device)
    v_cache = _randn((num_blocks, num_kv_heads, block_size, value_size), dtype, std, gen, device)
    new_k = _randn((num_seqs, num_kv_heads, head_size), dtype, std, gen, device)
    new_v = _randn((num_seqs, num_kv_heads, value_size), dtype, std, gen, device)
    return DecodeCase(
        name=name, dtype=dtype, num_heads=num_heads, num_kv_heads=num_kv_heads, head_size=head_size,
        block_size=block_size, scale=1.0 / math.sqrt(head_size),
        q=q, k_cache=k_cache, v_cache=v_cache,
        block_tables=block_tables.to(device), seq_lens=seq_lens.to(device),
        new_k=new_k, new_v=new_v, slot_mapping=slot_mapping.to(device),
    )


def _cpu_gen(seed):
    g = torch.Generator()
    g.manual_seed(seed)
    return g


def config1_small(seed=1, device="cpu") -> DecodeCase:
    """fp16, 4 sequences, 8 q-heads / 2 kv-heads, head 64, block 16, 128-block pool, lengths U[1,256]."""
    lens = torch.randint(1, 257, (4,), generator=_cpu_gen(seed))
    return build_case("c1_small_fp16", dtype=torch.float16, seq_lens=lens, num_heads=8, num_kv_heads=2, head_size=64,
                      block_size=16, num_blocks=128, max_blocks_per_seq=16, seed=seed, device=device)


def config2_llama8b(seed=2, device="cuda", num_seqs=64, seq_len=4096) -> DecodeCase:
    """bf16, batch 64, 32/8 heads, head 128, block 16, every length 4096, tables = permutation of a
    16384-block pool (the pool is exactly full)."""
    lens = torch.full((num_seqs,), seq_len, dtype=torch.int64)
    return build_case("c2_llama3_8b_bf16", dtype=torch.bfloat16, seq_lens=lens, num_heads=32, num_kv_heads=8,
                      head_size=128, block_size=16, num_blocks=num_seqs * ((seq_len + 15) // 16), seed=seed, device=device)


def config3_lengths(seed=3, num_seqs=256, lo=16, hi=32768) -> torch.Tensor:
    """Log-uniform sequence lengths of the ragged configuration."""
    u = torch.rand(num_seqs, generator=_cpu_gen(seed))
    return torch.exp(math.log(lo) + u * (math.log(hi) - math.log(lo))).round().to(torch.int64).clamp(lo, hi)


def config3_ragged72b(seed=3, device="cuda", num_seqs=256, lo=16, hi=32768) -> DecodeCase:
    """bf16, batch 256, 64/8 heads, head 128, lengths log-uniform in [16, 32768], N(0, 0.5) data."""
    lens = config3_lengths(seed, num_seqs, lo, hi)
    return build_case("c3_ragged_72b_bf16", dtype=torch.bfloat16, seq_lens=lens, num_heads=64, num_kv_heads=8,
                      head_size=128, block_size=16, max_blocks_per_seq=(hi + 15) // 16, std=0.5, seed=seed,
                      device=device, slack_blocks=64)


def config4_longctx(seed=4, device="cuda", num_seqs=2, seq_len=131072) -> DecodeCase:
    """fp16, batch 2, 32/8 heads, head 128, both sequences 131072 tokens."""
    lens = torch.full((num_seqs,), seq_len, dtype=torch.int64)
    return build_case("c4_longctx_fp16", dtype=torch.float16, seq_lens=lens, num_heads=32, num_kv_heads=8,
                      head_size=128, block_size=16, seed=seed, device=device)


def config5_lengths(seed=5, num_seqs=2048, lo=1024, hi=8192) -> torch.Tensor:
    """Lengths of the 2048-sequence batch; the same on every rank so shards are consistent."""
    return torch.randint(lo, hi + 1, (num_seqs,), generator=_cpu_gen(seed))


def config5_shard(rank=0, world=1, seed=5, device="cuda", num_seqs=2048) -> DecodeCase:
    """bf16, 64/8 heads, head 128; sequence i of the 2048 goes to rank i % world, each rank with its
    own pool and tables (no inter-GPU traffic)."""
    lens = config5_lengths(seed, num_seqs)[rank::world]
    return build_case(f"c5_shard{rank}of{world}_bf16", dtype=torch.bfloat16, seq_lens=lens, num_heads=64,
                      num_kv_heads=8, head_size=128, block_size=16, max_blocks_per_seq=8192 // 16,
                      seed=seed * 1000 + rank, device=device)


# ---- prefill ------------------------------------------------------------------------------------

@dataclass
class PrefillCase:
    name: str
    dtype: torch.dtype
    num_heads: int
    num_kv_heads: int
    head_size: int
    block_size: int
    scale: float
    q: torch.Tensor               # [total_q, num_heads, head_size], packed over sequences
    k_cache: torch.Tensor         # pools already hold every token, the new ones included
    v_cache: torch.Tensor
    block_tables: torch.Tensor    # [num_seqs, max_blocks_per_seq]
    seq_lens: torch.Tensor        # [num_seqs] total KV length (cached + new)
    cum_seq_lens_q: torch.Tensor  # [num_seqs + 1]

    @property
    def num_seqs(self) -> int:
        return self.seq_lens.numel()

    @property
    def flops(self) -> int:
        """2 * 2 * heads * head_size * (number of (query, key) pairs the causal mask keeps)."""
        new = (self.cum_seq_lens_q[1:] - self.cum_seq_lens_q[:-1]).double()
        total = self.seq_lens.double()
        pairs = (new * (total - new) + new * (new + 1) / 2).sum().item()
        return int(4 * self.num_heads * self.head_size * pairs)

    def to(self, device) -> "PrefillCase":
        moved = {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in self.__dict__.items()}
        return PrefillCase(**moved)


def build_prefill_case(name, *, dtype, new_lens, cached_lens, num_heads, num_kv_heads, head_size, block_size,
                       std=1.0, seed=0, device="cpu", value_size=None, index_dtype=torch.int64) -> PrefillCase:
    """One prefill problem: sequence i has cached_lens[i] tokens in the cache and new_lens[i] new query
    tokens (whose K/V are in the cache as well, as after paged_caching)."""
    new_lens = torch.as_tensor(new_lens, dtype=torch.int64)
    cached_lens = torch.as_tensor(cached_lens, dtype=torch.int64)
    base = build_case(name, dtype=dtype, seq_lens=new_lens + cached_lens, num_heads=num_heads, num_kv_heads=num_kv_heads,
                      head_size=head_size, block_size=block_size, std=std, seed=seed, device=device, value_size=value_size)
    gen = torch.Generator(device=torch.device(device))
    gen.manual_seed(seed + 17)
    total_q = int(new_lens.sum())
    q = _randn((total_q, num_heads, head_size), dtype, std, gen, torch.device(device))
    cum = torch.zeros(new_lens.numel() + 1, dtype=torch.int64)
    cum[1:] = torch.cumsum(new_lens, 0)
    return PrefillCase(name=name, dtype=dtype, num_heads=num_heads, num_kv_heads=num_kv_heads, head_size=head_size,
                       block_size=block_size, scale=base.scale, q=q, k_cache=base.k_cache, v_cache=base.v_cache,
                       block_tables=base.block_tables.to(index_dtype), seq_lens=base.seq_lens.to(index_dtype),
                       cum_seq_lens_q=cum.to(index_dtype).to(device))


def prefill_llama8b(seed=6, device="cuda", num_seqs=8, new_len=2048, cached_len=0) -> PrefillCase:
    """Llama-3-8B-shape prefill: bf16, 32/8 heads, head 128, block 16, `num_seqs` prompts of `new_len` tokens."""
    return build_prefill_case("prefill_llama3_8b_bf16", dtype=torch.bfloat16, new_lens=[new_len] * num_seqs,
                              cached_lens=[cached_len] * num_seqs, num_heads=32, num_kv_heads=8, head_size=128,
                              block_size=16, seed=seed, device=device)
