"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

Real Mixtral / Qwen3 / DeepSeek checkpoints are not available offline; these generators stand in for them.

Expert weights come from a counter-based generator, so that any expert of any layer can be produced
independently, on the host with numpy (`make_expert_blob`, what the CPU oracle reads) or directly in device
memory with torch (`make_expert_blobs_torch`, what a deep resident stack is filled from) -- same bytes:

  key(seed, layer, expert, projection) = mix(mix(mix(mix(seed) + layer) + expert) + projection)
  word(b, i)                           = mix(key + b * 8 + i)            b = block index, i = 0..7
  mix                                  = splitmix64 finaliser

  Q4_0 block b: quant bytes 0..15 = the bytes of word(b, 0), word(b, 1) (two uniform nibbles per byte);
                scale = f16(0.002 + u * 0.008),  u = (word(b, 7) >> 40) / 2^24
  Q8_0 block b: quant bytes 0..31 = the bytes of word(b, 0..3) as int8; a byte that comes out as -128 is
                replaced by ((word(b, 4) >> byte index) & 0xFFFF) % 255 - 127, so that values lie in [-127, 127];
                scale = f16(0.0005 + u * 0.0015)

Router matrices and activations are numpy draws:
  router       : default_rng([seed, layer, 1 << 20]).normal(0, 0.02, (E, D)) as f32
  activations  : default_rng([seed, 1 << 21, batch]).standard_normal((B, D)) as f32
"""
from dataclasses import dataclass

import numpy as np

Q4_0, Q8_0 = 0, 1
BLOCK_BYTES = {Q4_0: 18, Q8_0: 34}
SCALE_RANGE = {Q4_0: (0.002, 0.01), Q8_0: (0.0005, 0.002)}


@dataclass(frozen=True)
class MoeShape:
    name: str
    dtype: int
    d_model: int
    d_ff: int
    num_experts: int
    top_k: int
    seed: int
    scoring: int = 0          # 0 softmax, 1 sigmoid
    n_group: int = 1
    topk_group: int = 1
    scaling: float = 1.0
    shared: bool = False
    layers: int = 1


CONFIGS = {
    # the five benchmark configurations (shapes only; batch sizes are chosen by the caller)
    "cfg0-mixtral-q4_0": MoeShape("cfg0-mixtral-q4_0", Q4_0, 4096, 14336, 8, 2, seed=0),
    "cfg1-qwen3-q8_0": MoeShape("cfg1-qwen3-q8_0", Q8_0, 2048, 768, 128, 8, seed=1),
    "cfg2-mixtral-stack-q4_0": MoeShape("cfg2-mixtral-stack-q4_0", Q4_0, 4096, 14336, 8, 2, seed=0, layers=32),
    "cfg3-qwen3-prefill-q8_0": MoeShape("cfg3-qwen3-prefill-q8_0", Q8_0, 2048, 768, 128, 8, seed=1, layers=48),
    "cfg4-deepseek-v3-q4_0": MoeShape("cfg4-deepseek-v3-q4_0", Q4_0, 7168, 2048, 256, 8, seed=0, scoring=1, n_group=8,
                                      topk_group=4, scaling=2.5, shared=True, layers=58),
}


def expert_bytes(dtype, d_model, d_ff):
    return 3 * ((d_model * d_ff + 31) // 32) * BLOCK_BYTES[dtype]


# ------------------------------------------------------------------ counter-based generator
_M64 = (1 << 64) - 1
_GOLDEN, _C1, _C2 = 0x9E3779B97F4A7C15, 0xBF58476D1CE4E5B9, 0x94D049BB133111EB


def _mix_int(x):
    z = (x + _GOLDEN) & _M64
    z = ((z ^ (z >> 30)) * _C1) & _M64
    z = ((z ^ (z >> 27)) * _C2) & _M64
    return z ^ (z >> 31)


def projection_key(seed, layer, expert, projection):
    k = _mix_int(seed & _M64)
    for v in (layer, expert, projection):
        k = _mix_int((k + v) & _M64)
    return k


def _mix_np(x):
    with np.errstate(over="ignore"):
        z = x + np.uint64(_GOLDEN)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(_C1)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(_C2)
        return z ^ (z >> np.uint64(31))


def make_projection(dtype, n_weights, key):
    """One projection's block stream (uint8) for the generator key `key` (numpy)."""
    n_blocks = (n_weights + 31) // 32
    nq = 2 if dtype == Q4_0 else 4
    with np.errstate(over="ignore"):
        base = np.uint64(key) + np.arange(n_blocks, dtype=np.uint64) * np.uint64(8)
        words = _mix_np(base[:, None] + np.arange(nq, dtype=np.uint64)[None, :])
        w7 = _mix_np(base + np.uint64(7))
    lo, hi = SCALE_RANGE[dtype]
    u = (w7 >> np.uint64(40)).astype(np.uint32).astype(np.float32) * np.float32(2.0 ** -24)  # 24 bits: exact in f32
    scales = (np.float32(lo) + u * np.float32(hi - lo)).astype(np.float16)
    out = np.empty((n_blocks, BLOCK_BYTES[dtype]), np.uint8)
    out[:, :2] = scales.view(np.uint8).reshape(n_blocks, 2)
    q = words.view(np.uint8).reshape(n_blocks, nq * 8)  # little-endian bytes of the words
    if dtype == Q8_0:
        r, c = np.nonzero(q == 0x80)  # about one byte in 256
        if r.size:
            with np.errstate(over="ignore"):
                w4 = _mix_np(base[r] + np.uint64(4))
            alt = ((w4 >> c.astype(np.uint64)) & np.uint64(0xFFFF)) % np.uint64(255)
            q = q.copy()
            q[r, c] = (alt.astype(np.int16) - 127).astype(np.int8).view(np.uint8)
    out[:, 2:] = q
    return out.reshape(-1)


def make_expert_blob(dtype, d_model, d_ff, seed, layer=0, expert=0):
    """One gate||up||down block stream (inference.rs:1096-1114 layout)."""
    return np.concatenate([make_projection(dtype, d_model * d_ff, projection_key(seed, layer, expert, p)) for p in range(3)])


def _signed(v):
    return v - (1 << 64) if v >= (1 << 63) else v


def make_expert_blobs_torch(dtype, d_model, d_ff, seed, layer, experts, device):
    """The blobs of `experts` (a list of expert indices of `layer`) as one uint8 tensor [len(experts), expert_bytes]
    on `device`: the same bytes as make_expert_blob, computed with 64-bit integer tensor arithmetic."""
    import torch
    n_blocks = (d_model * d_ff + 31) // 32
    nq = 2 if dtype == Q4_0 else 4
    bb = BLOCK_BYTES[dtype]
    keys = torch.tensor([[_signed(projection_key(seed, layer, e, p)) for p in range(3)] for e in experts], dtype=torch.int64,
                        device=device)  # [n, 3]

    def srl(z, s):
        return (z >> s) & ((1 << (64 - s)) - 1)

    def mix(x):
        z = x + _signed(_GOLDEN)
        z = (z ^ srl(z, 30)) * _signed(_C1)
        z = (z ^ srl(z, 27)) * _signed(_C2)
        return z ^ srl(z, 31)

    base = keys[:, :, None] + torch.arange(n_blocks, dtype=torch.int64, device=device)[None, None, :] * 8  # [n, 3, blocks]
    out = torch.empty((len(experts), 3, n_blocks, bb), dtype=torch.uint8, device=device)
    lo, hi = SCALE_RANGE[dtype]
    u = srl(mix(base + 7), 40).to(torch.float32) * (2.0 ** -24)
    f32 = dict(dtype=torch.float32, device=device)
    scales = (torch.tensor(float(np.float32(lo)), **f32) + u * torch.tensor(float(np.float32(hi - lo)), **f32)).to(torch.float16)
    out[..., :2] = scales.view(torch.uint8).reshape(len(experts), 3, n_blocks, 2)
    shifts = torch.arange(8, dtype=torch.int64, device=device) * 8
    for i in range(nq):
        w = mix(base + i)
        out[..., 2 + 8 * i:10 + 8 * i] = ((w[..., None] >> shifts) & 0xFF).to(torch.uint8)
    if dtype == Q8_0:
        w4 = mix(base + 4)
        sh = torch.arange(32, dtype=torch.int64, device=device)
        # the low 16 bits after a shift by at most 31 are original bits: arithmetic and logical shifts agree on them
        alt = (((w4[..., None] >> sh) & 0xFFFF) % 255 - 127).to(torch.int8).view(torch.uint8)
        q = out[..., 2:]
        out[..., 2:] = torch.where(q == 0x80, alt, q)
    return out.reshape(len(experts), 3 * n_blocks * bb)


def make_router(num_experts, d_model, seed, layer=0):
    return np.random.default_rng([seed, layer, 1 << 20]).normal(0.0, 0.02, (num_experts, d_model)).astype(np.float32)


def make_activations(n_tokens, d_model, seed, batch=0):
    return np.random.default_rng([seed, 1 << 21, batch]).standard_normal((n_tokens, d_model)).astype(np.float32)


def zipf_logit_bias(num_experts, s, seed, layer=0, strength=1.0):
    """Routing-locality skew: expert of popularity rank r gets logit bias -strength*s*ln(r+1), ranks
    shuffled per layer (the reference's Zipf workloads use w_r = 1/(r+1)^s, workload.rs:60-140)."""
    rng = np.random.default_rng([seed, layer, 1 << 22])
    ranks = rng.permutation(num_experts)
    return (-strength * s * np.log(ranks + 1.0)).astype(np.float32)
