"""Key/value cache metadata of the reference's HAL (crates/hal/src/lib.rs:129-239): how large the device buffers are, where an
element lives, and which absolute positions the cached window covers.  Host bookkeeping only; the device buffers themselves
belong to the model (sptorch_ext_gpt_enable_kv_cache) and use the same [layer, position, head, dim] order per sequence."""
from __future__ import annotations

from dataclasses import dataclass

_DTYPE_BYTES = {"F32": 4, "F16": 2, "BF16": 2}


@dataclass(frozen=True)
class KvCacheBufferSpec:
    device: tuple          # (backend name, ordinal), the reference's DeviceId
    dtype: str             # "F32" | "F16" | "BF16"
    n_layer: int
    max_context: int
    n_head: int
    head_dim: int

    def __post_init__(self):
        if self.max_context <= 0:
            raise ValueError("max_context must be positive")
        if self.n_head <= 0:
            raise ValueError("n_head must be positive")
        if self.head_dim <= 0:
            raise ValueError("head_dim must be positive")
        if self.dtype not in _DTYPE_BYTES:
            raise ValueError(f"unknown dtype {self.dtype}")

    def elements_per_kind(self) -> int:
        return self.n_layer * self.max_context * self.n_head * self.head_dim

    def total_elements(self) -> int:
        return 2 * self.elements_per_kind()

    def total_bytes(self) -> int:
        return self.total_elements() * _DTYPE_BYTES[self.dtype]

    def element_offset(self, layer: int, position: int, head: int, dim: int) -> int:
        """Linear element offset inside one K or V buffer; ``position`` is a slot of the window, not an absolute position."""
        for name, v, hi in (("layer", layer, self.n_layer), ("position", position, self.max_context),
                            ("head", head, self.n_head), ("dim", dim, self.head_dim)):
            if not 0 <= v < hi:
                raise IndexError(f"{name} out of range")
        return ((layer * self.max_context + position) * self.n_head + head) * self.head_dim + dim


@dataclass
class KvCacheWindowState:
    max_context: int
    window_start: int = 0
    cached_len: int = 0

    def __post_init__(self):
        if self.max_context <= 0:
            raise ValueError("max_context must be positive")

    def next_position(self) -> int:
        return self.window_start + self.cached_len

    def last_position(self):
        return None if self.cached_len == 0 else self.window_start + self.cached_len - 1

    def prefill(self, start_position: int, length: int) -> None:
        if length > self.max_context:
            raise ValueError("prefill len cannot exceed max_context")
        self.window_start, self.cached_len = start_position, length

    def append(self, length: int) -> None:
        total = self.cached_len + length
        self.window_start += max(0, total - self.max_context)
        self.cached_len = min(total, self.max_context)


def spec_of(model, max_context: int | None = None) -> KvCacheBufferSpec:
    """The spec of a device model's cache (GPT::kv_cache_spec, crates/nn/src/lib.rs:1531-1538)."""
    from .backend import BF16
    c = model.cfg
    return KvCacheBufferSpec(("cuda", model.b.lib.sptorch_ext_device()), "BF16" if model.dtype == BF16 else "F32", c["n_layer"],
                             max_context or c["seq_len"], c["n_head"], c["d_model"] // c["n_head"])
