"""Descriptions of a model as data: which parts each layer is made of, with every size
and constant as a parameter, and the order in which layers run.

A *spec* is a frozen dataclass with a `kind` string.  The part registries
(`llmgen_b200.parts.registry`) map a kind to the class that runs it on the GPU, so a new
mixer, feed-forward, norm or position encoding is one spec class, one runtime class and one
`register_*` call; nothing in the engine or the cache manager changes.

The reference builds the same tree from `Ctx.config_params` and weights found by spec key
(src/module/module.zig:32-83, src/models/qwen3.zig:142-340).  Its modules append graph
nodes; ours hold device weights and launch kernels.  Tensor names are parameters of the
specs, given by the architecture's builder, so no part knows which model it is in.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple

# How a declared tensor is kept on the device, and how the random-weights mode draws it.
MATRIX = "matrix"      # projection or table of embeddings: compute dtype (bf16 or fp32)
VECTOR = "vector"      # norm gains and other small vectors: always fp32 on the device
INT_TABLE = "int_table"  # integer tables: int32

INIT_NORMAL = "normal"              # N(0, sigma)
INIT_ONE_PLUS_NORMAL = "one_plus"   # 1 + N(0, sigma_norm)


@dataclass(frozen=True)
class WeightDecl:
    """One tensor a part reads from the model file."""
    name: str
    shape: Tuple[int, ...]
    kind: str = MATRIX
    init: str = INIT_NORMAL


# ----------------------------------------------------------------------------- norms
@dataclass(frozen=True)
class RMSNormSpec:
    """y = x * rsqrt(mean(x^2) + eps) * (weight + weight_offset) over the last `dim` values.

    Reference: src/module/norm.zig:49-86, src/backend/cpu/norm.zig:60-93.
    """
    dim: int
    eps: float
    weight: str
    weight_offset: float = 0.0
    kind: str = "rmsnorm"


# ----------------------------------------------------------------- position encodings
@dataclass(frozen=True)
class RopeSpec:
    """Rotary position encoding over the first `rotary_dim` values of a head, angle =
    pos / theta^(2i/rotary_dim).  `pairing` says which two values are turned together: "half" is the
    half-split (NEOX) pairing (i, i + rotary_dim/2) of the reference; the attention kernels are told
    the pairing and refuse one they do not implement.

    Reference: src/module/rope.zig:60-107, src/backend/cpu/rope.zig:13-75.
    """
    rotary_dim: int
    theta: float
    max_positions: int
    pairing: str = "half"
    kind: str = "rope"


# ----------------------------------------------------------------------------- mixers
@dataclass(frozen=True)
class AttentionSpec:
    """Causal grouped-query attention over a paged key/value cache.

    q = x Wq^T, k = x Wk^T, v = x Wv^T (no bias); optional RMSNorm over each head of q and
    of k (one gain vector shared by all heads) before the position encoding; softmax of
    q.k * scale over keys 0..pos (or the last `window` of them); output projection Wo.

    Reference: src/models/qwen3.zig:165-209, src/module/attention.zig:85-92,
    src/backend/cpu/attention.zig:64-118.
    """
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    q_proj: str
    k_proj: str
    v_proj: str
    o_proj: str
    q_norm: Optional[RMSNormSpec] = None
    k_norm: Optional[RMSNormSpec] = None
    position: Optional[RopeSpec] = None
    window: Optional[int] = None
    kind: str = "attention"


# ---------------------------------------------------------------------- feed-forwards
@dataclass(frozen=True)
class GatedMLPSpec:
    """Dense gated feed-forward: down( act(x Wg^T) * (x Wu^T) ).

    Reference: src/models/qwen3.zig:142-163 (SwiGLU: act = x / (1 + exp(-x)),
    src/backend/cpu/activation.zig:13-17).
    """
    hidden_size: int
    intermediate_size: int
    gate_proj: str
    up_proj: str
    down_proj: str
    activation: str = "silu"
    kind: str = "gated_mlp"


# ----------------------------------------------------------------------------- blocks
@dataclass(frozen=True)
class PreNormBlockSpec:
    """x1 = x + mixer(norm(x)); x2 = x1 + ffn(norm(x1)).

    Reference: src/models/qwen3.zig:211-237.
    """
    mixer_norm: object
    mixer: object
    ffn_norm: object
    ffn: object
    kind: str = "prenorm"


@dataclass(frozen=True)
class RunItem:
    """One entry of the run list: run `layer`, with cache number `cache`.

    A layer may be named by several items (each with a cache of its own or a shared one),
    and an item with `writes_cache=False` reads the cache that another item filled in the
    same step.  `cache` is None for a layer that keeps nothing between steps.
    """
    layer: int
    cache: Optional[int]
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    """A whole decoder: embedding, layers, run list, final norm, output projection."""
    architecture: str
    vocab_size: int
    hidden_size: int
    embedding: str                       # name of the [vocab, hidden] table
    layers: Tuple[object, ...]           # block specs
    run_order: Tuple[RunItem, ...]
    final_norm: object
    lm_head: str                         # same name as `embedding` when tied
    max_positions: int
    eos_token_ids: Tuple[int, ...] = ()
    init_sigma: float = 0.02             # defaults of the random-weights mode
    init_sigma_norm: float = 0.1
    embedding_scale: float = 1.0         # rows of the table are multiplied by this as they enter the residual
    logit_cap: float = 0.0               # > 0: logits = cap * tanh(logits / cap)
    # Tensors that a model folder of this architecture may carry although the model reads none of them
    # (shell patterns), and (name, declared name) pairs of such tensors that must then hold the same values.
    ignorable_tensors: Tuple[str, ...] = ()
    same_as: Tuple[Tuple[str, str], ...] = ()

    @property
    def tied(self) -> bool:
        return self.lm_head == self.embedding


def default_run_order(num_layers: int) -> Tuple[RunItem, ...]:
    return tuple(RunItem(layer=i, cache=i) for i in range(num_layers))
