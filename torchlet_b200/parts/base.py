"""Interfaces of the parts a layer is put together from, and their registries.

A part knows its own sizes and constants (from its ``PartSpec``) and the names of
its own tensors below a prefix.  It does not know which model it is in, which layer
it is, or what stands before or after it.  The reference has the same parts as
``nn.Module`` classes with constructor arguments
(v10_triton_paged_gqa/layer/{gqa,ffn_swiglu,rms_norm,rope,transformer_block}.py);
here each kind is looked up by name so that a layer may choose any of them.

Data contract of a step (``StepContext`` in ``torchlet_b200.engine.batch``):

* ``x``   : the normed input of a sub-layer, ``[T, hidden]`` in the compute dtype;
* ``acc`` : the residual stream, ``[T, hidden]`` in float32.  A mixer or a
  feed-forward ADDS its output into ``acc``; the residual sum is therefore always
  taken in 32-bit.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

from ..config.spec import PartSpec


@dataclass(frozen=True)
class TensorSpec:
    """A tensor a part expects in the checkpoint."""

    name: str
    shape: tuple
    init: str = "normal"  # "normal": N(0, std); "ones": 1 + N(0, norm_std)
    optional: bool = False


@dataclass(frozen=True)
class KVSpec:
    """Per-token history a mixer keeps in pages: keys and values of every token,
    or of the last ``window`` tokens only."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None

    def group_key(self) -> tuple:
        return (self.num_kv_heads, self.head_dim, self.window)


@dataclass(frozen=True)
class StateSpec:
    """Fixed-size state a mixer keeps per live request (one row per slot),
    zeroed when a request is admitted."""

    shape: tuple
    dtype: str = "float32"


class Part:
    """Base of all parts.  Sub-classes set ``kind`` and implement what applies."""

    kind: str = ""

    def __init__(self, spec: PartSpec):
        self.spec = spec

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        return []

    def load(self, tensors: dict, prefix: str, device, dtype) -> None:
        """Take this part's tensors (by full name) and lay them out for its kernels."""


class Norm(Part):
    """A norm reads rows of the float32 stream ``acc`` and returns them normed in the compute
    dtype.  A sub-class implements ``forward``; blocks and the model call ``apply``, which first
    completes any sum into ``acc`` that a product left unfinished, so that ``forward`` can read
    ``acc`` as it stands.  A norm that can take over such a sum and finish it inside its own
    kernel sets ``fuses_pending`` and asks ``ctx.take_pending(acc)`` itself."""

    fuses_pending = False

    def apply(self, ctx, acc, out=None, rows=None, name="normed"):
        if not self.fuses_pending:
            ctx.flush_pending()
        return self.forward(ctx, acc, out=out, rows=rows, name=name)

    def forward(self, ctx, acc, out=None, rows=None, name="normed"):
        """Return the normed ``acc`` rows (all, or those ``rows`` names, int32) in the compute
        dtype; ``out`` or a buffer called ``name`` receives them."""
        raise NotImplementedError


class Positions(Part):
    """A position encoding applied inside a mixer: ``encode(ctx, qkv, num_heads, num_kv_heads)``
    changes the q and k heads of the fused ``qkv`` rows in place; the mixer then stores k and v
    itself.  An encoding that can write k and v to the cache pages in the same pass sets
    ``stores_kv`` and implements ``encode_and_store(ctx, qkv, num_heads, num_kv_heads, cache)``
    instead.  ``graph_safe`` False keeps a model that uses it out of the captured decode graph
    (it plans on the host)."""

    graph_safe = True
    stores_kv = False

    def encode(self, ctx, qkv, num_heads, num_kv_heads) -> None:
        raise NotImplementedError


class Mixer(Part):
    def kv_spec(self) -> Optional[KVSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def forward(self, ctx, x, acc, cache) -> None:
        """Mix ``x`` over each request's history and add the result into ``acc``.

        ``cache`` is the ``LayerCache`` of this execution: pages and block table if
        ``kv_spec`` is set, the state rows if ``state_spec`` is set, and
        ``cache.writable`` False when the execution reads another's cache.
        """
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx, x, acc) -> None:
        """Add the feed-forward of ``x`` into ``acc``."""
        raise NotImplementedError


class Block:
    """An arrangement of a layer's parts around the residual stream.  ``norm_roles`` names the
    norms the arrangement needs; the layer's description must hold one for each role, and
    ``norms`` maps the roles to the built parts."""

    kind: str = ""
    norm_roles: tuple = ()

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, norms: dict):
        missing = [role for role in self.norm_roles if role not in norms]
        if missing:
            raise ValueError(f"block arrangement {self.kind!r} needs norms for the roles {missing}")
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.norms = dict(norms)

    def forward(self, ctx, acc, cache) -> None:
        raise NotImplementedError


class _Registry:
    def __init__(self, what: str):
        self.what = what
        self._items: dict[str, type] = {}

    def register(self, name: str) -> Callable[[type], type]:
        def _do(cls: type) -> type:
            cls.kind = name
            self._items[name] = cls
            return cls

        return _do

    def get(self, name: str) -> type:
        try:
            return self._items[name]
        except KeyError:
            raise KeyError(
                f"unknown {self.what} {name!r}; registered: {', '.join(sorted(self._items)) or 'none'}"
            ) from None

    def names(self) -> list[str]:
        return sorted(self._items)


MIXERS = _Registry("mixer")
FEED_FORWARDS = _Registry("feed-forward")
NORMS = _Registry("norm")
POSITIONS = _Registry("position encoding")
BLOCKS = _Registry("block arrangement")


def build_part(registry: _Registry, spec: PartSpec) -> Part:
    return registry.get(spec.kind)(spec)
