"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

Real Mixtral / Qwen3 / DeepSeek checkpoints are not available offline; these generators stand in
for them.  Draw order (fixed, so every consumer sees the same bytes):
  expert blob  : rng = default_rng([seed, layer, expert]); for projection in gate, up, down:
                 scales = rng.uniform(lo, hi, n_blocks) -> f16;  quants = rng.integers(...) per block
  router       : default_rng([seed, layer, 1 << 20]).normal(0, 0.02, (E, D)) as f32
  activations  : default_rng([seed, 1 << 21, batch]).standard_normal((B, D)) as f32
"""
from dataclasses import dataclass

import numpy as np

Q4_0, Q8_0 = 0, 1
BLOCK_BYTES = {Q4_0: 18, Q8_0: 34}


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


def make_projection(dtype, n_weights, rng):
    n_blocks = (n_weights + 31) // 32
    out = np.empty((n_blocks, BLOCK_BYTES[dtype]), np.uint8)
    if dtype == Q4_0:
        scales = rng.uniform(0.002, 0.01, n_blocks).astype(np.float16)
        q = rng.integers(0, 16, (n_blocks, 32), dtype=np.uint8)
        out[:, 2:] = q[:, :16] | (q[:, 16:] << 4)
    else:
        scales = rng.uniform(0.0005, 0.002, n_blocks).astype(np.float16)
        out[:, 2:] = rng.integers(-127, 128, (n_blocks, 32), dtype=np.int8).view(np.uint8)
    out[:, :2] = scales.view(np.uint8).reshape(n_blocks, 2)
    return out.reshape(-1)


def make_expert_blob(dtype, d_model, d_ff, seed, layer=0, expert=0):
    """One gate||up||down block stream (inference.rs:1096-1114 layout)."""
    rng = np.random.default_rng([seed, layer, expert])
    return np.concatenate([make_projection(dtype, d_model * d_ff, rng) for _ in range(3)])


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
