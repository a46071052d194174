"""The reference's on-disk weight formats, read by the library's host-side readers (csrc/weights.cu): binary ``.sptc``
checkpoints, JSON ``state_dict`` files with their manifest, and safetensors (crates/serialize/src/lib.rs, safetensors.rs).
Reading needs no GPU; loading into a device model does."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib

AUTO, SPTC, STATE_DICT, SAFETENSORS = 0, 1, 2, 3


class WeightsError(RuntimeError):
    pass


class WeightFile:
    """An opened weight file: ``len()``, ``names()``, ``entry(i) -> (name, shape, stored dtype, float32 array)``."""

    def __init__(self, path: str, fmt: int = AUTO):
        self.lib = _lib.load()
        self.h = self.lib.sptorch_ext_weights_open(str(path).encode(), fmt)
        if not self.h:
            raise WeightsError(_lib.last_error())
        self.format = self.lib.sptorch_ext_weights_format(self.h)

    def close(self):
        if self.h:
            self.lib.sptorch_ext_weights_close(self.h)
            self.h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __len__(self):
        return int(self.lib.sptorch_ext_weights_count(self.h))

    def names(self):
        return [self.lib.sptorch_ext_weights_name(self.h, i).decode() for i in range(len(self))]

    def entry(self, i: int):
        L = self.lib
        shape = tuple(int(L.sptorch_ext_weights_dim(self.h, i, k)) for k in range(L.sptorch_ext_weights_ndim(self.h, i)))
        n = int(L.sptorch_ext_weights_numel(self.h, i))
        data = np.ctypeslib.as_array(L.sptorch_ext_weights_data(self.h, i), shape=(n,)).copy() if n else np.zeros(0, np.float32)
        return (L.sptorch_ext_weights_name(self.h, i).decode(), shape, L.sptorch_ext_weights_dtype(self.h, i).decode(), data)

    def get(self, name: str):
        for i, n in enumerate(self.names()):
            if n == name:
                return self.entry(i)
        return None


def load_into(model, path: str, fmt: int = AUTO, mapping=None):
    """Checks the file against the model's named parameters with the reference's strictness and uploads it.
    ``mapping`` (safetensors only): {model parameter name: name in the file}, as SafeTensorsFile::load_into."""
    with WeightFile(path, fmt) as w:
        arr, n = None, 0
        if mapping:
            flat = []
            for k, v in mapping.items():
                flat += [k.encode(), v.encode()]
            arr, n = (C.c_char_p * len(flat))(*flat), len(mapping)
        if model.b.lib.sptorch_ext_gpt_load_weights(model.h, w.h, arr, n):
            raise WeightsError(_lib.last_error())


def load_bundle(model, weights_path: str):
    """JSON state_dict + ``<path>.manifest.json`` (load_state_dict_bundle, crates/serialize/src/lib.rs:366-441)."""
    if model.b.lib.sptorch_ext_gpt_load_bundle(model.h, str(weights_path).encode()):
        raise WeightsError(_lib.last_error())


def model_parameters(model):
    """[(name, shape)] of the device model in the reference's named_parameters order, as the library reports them."""
    L = model.b.lib
    out = []
    for i in range(L.sptorch_ext_gpt_param_count(model.h)):
        name = C.create_string_buffer(128)
        dims = (C.c_size_t * 8)()
        nd = C.c_size_t(8)
        if L.sptorch_ext_gpt_param_info(model.h, i, name, 128, dims, C.byref(nd)):
            raise WeightsError(_lib.last_error())
        out.append((name.value.decode(), tuple(int(dims[k]) for k in range(nd.value))))
    return out
