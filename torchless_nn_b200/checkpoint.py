"""Weight interchange with the reference's on-disk format.

The reference has no checkpoint code in the library; its notebook pickles one entry per layer,
``[{"name": type(layer).__name__, "parameters": [ndarray, ...]}, ...]`` (demo.ipynb, ``save_weights``), and loads it
back in place with ``parameter *= 0; parameter += xp.array(arr)`` (``load_weights``).  The two functions here read and
write exactly that layout, so a checkpoint written by the reference runs on this engine and the other way round.  The
tied token table is registered by ``GPTEmbedFront`` only, so the ``GPTEmbedBack`` entry of a file has no arrays.

The file is a pickle: loading goes through an unpickler that only admits NumPy arrays, dtypes and plain containers,
so a checkpoint cannot run code when it is opened.
"""
from __future__ import annotations

import pickle

import numpy as np

_ALLOWED = {
    ("numpy.core.multiarray", "_reconstruct"), ("numpy._core.multiarray", "_reconstruct"),
    ("numpy", "ndarray"), ("numpy", "dtype"),
    ("numpy.core.multiarray", "scalar"), ("numpy._core.multiarray", "scalar"),
    ("numpy.core.numeric", "_frombuffer"), ("numpy._core.numeric", "_frombuffer"),
}


class _ArraysOnly(pickle.Unpickler):
    def find_class(self, module, name):
        if (module, name) in _ALLOWED:
            return super().find_class(module, name)
        raise pickle.UnpicklingError(f"checkpoint refers to {module}.{name}; only NumPy arrays are accepted")


def read_checkpoint(path) -> list:
    """The file's list of ``{"name", "parameters"}`` entries, validated."""
    with open(path, "rb") as handle:
        entries = _ArraysOnly(handle).load()
    if not isinstance(entries, list):
        raise ValueError("checkpoint: expected a list with one entry per layer")
    for e in entries:
        if not (isinstance(e, dict) and isinstance(e.get("name"), str) and isinstance(e.get("parameters"), list)):
            raise ValueError("checkpoint: every entry needs a 'name' and a list of 'parameters'")
        for a in e["parameters"]:
            if not isinstance(a, np.ndarray):
                raise ValueError("checkpoint: parameters must be NumPy arrays")
    return entries


def save_weights(model, path) -> None:
    """demo.ipynb ``save_weights``: one entry per layer, parameters copied to the host in registration order."""
    entries = []
    for layer in model.layers:
        entries.append({"name": type(layer).__name__, "parameters": [np.asarray(p.get()) for p in layer.parameters]})
    with open(path, "wb") as handle:
        pickle.dump(entries, handle)


def load_weights(model, path, strict: bool = True) -> None:
    """demo.ipynb ``load_weights``: overwrite the parameters of ``model.layers`` in place, layer by layer.

    The reference zips layers with entries silently; with ``strict`` (default) a different number of layers, layer
    class name, parameter count or shape raises ``ValueError`` instead of loading a prefix."""
    entries = read_checkpoint(path)
    layers = list(model.layers)
    if strict and len(entries) != len(layers):
        raise ValueError(f"checkpoint has {len(entries)} layers, the model has {len(layers)}")
    for layer, entry in zip(layers, entries):
        if strict and entry["name"] != type(layer).__name__:
            raise ValueError(f"checkpoint layer {entry['name']!r} does not match model layer {type(layer).__name__!r}")
        if strict and len(entry["parameters"]) != len(layer.parameters):
            raise ValueError(f"{entry['name']}: {len(entry['parameters'])} arrays for {len(layer.parameters)} parameters")
        for parameter, arr in zip(layer.parameters, entry["parameters"]):
            if tuple(parameter.shape) != tuple(arr.shape):
                raise ValueError(f"{entry['name']}: array of shape {arr.shape} for a parameter of shape {parameter.shape}")
            parameter[...] = np.asarray(arr, dtype=np.float32)
