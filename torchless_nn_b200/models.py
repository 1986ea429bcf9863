"""Layer lists of the benchmark configurations, built from this package's drop-in layers.

``build_network`` follows the reference notebook's recipes (final LayerNorm before the head: demo.ipynb:1209,1497):
GPT = [GPTEmbedFront, decoder TransformerBlock x L, LayerNorm, GPTEmbedBack | Dense]; ViT = [VitProjector,
encoder TransformerBlock x L, LayerNorm, VitMLPHead].  ``load_params`` writes a flat canonical parameter list
(``workloads.seeded_params``) into a network in place, visiting every distinct array once in registration order -
the same walk the golden-fixture generator performs on the reference's network.
"""
from __future__ import annotations

from . import workloads as wl


def build_network(spec, activation=None):
    from .network import Network
    from .layers import TransformerBlock, LayerNorm, Dense
    from .activations import GeLU
    from .transformer_adapters import (GPTEmbeddingTable, GPTEmbedFront, GPTEmbedBack, VitProjector, VitMLPHead)
    act = activation or GeLU
    if spec.kind == "gpt":
        tab = GPTEmbeddingTable(spec.vocab, spec.d_model)
        layers = [GPTEmbedFront(tab, spec.context)]
        layers += [TransformerBlock(spec.d_model, spec.context, spec.heads, act, decoder=True)
                   for _ in range(spec.layers)]
        layers.append(LayerNorm(spec.d_model))
        layers.append(GPTEmbedBack(tab) if spec.tied_head else Dense(spec.d_model, spec.vocab))
    else:
        layers = [VitProjector(tuple(spec.image), tuple(spec.patch), spec.d_model, spec.registers)]
        layers += [TransformerBlock(spec.d_model, 0, spec.heads, act) for _ in range(spec.layers)]
        layers += [LayerNorm(spec.d_model), VitMLPHead(spec.d_model, spec.classes)]
    return Network(layers)


def load_params(net, params) -> None:
    seen, it = set(), iter(params)
    for layer in net.layers:
        for p in layer.parameters:
            if id(p) in seen:
                continue
            seen.add(id(p))
            src = next(it)
            if tuple(p.shape) != tuple(src.shape):
                raise ValueError(f"parameter shape {p.shape} does not match the loaded array {src.shape}")
            p[...] = src
    if next(it, None) is not None:
        raise ValueError("more arrays than parameters")
    net.set_eval(True)


def build_seeded(name_or_spec, seed: int = wl.WEIGHT_SEED):
    """Network of a named configuration with the canonical seeded weights, arithmetic mode set to the spec's."""
    from . import backend
    spec = wl.CONFIGS[name_or_spec] if isinstance(name_or_spec, str) else name_or_spec
    backend.set_precision(spec.precision)
    net = build_network(spec)
    load_params(net, wl.seeded_params(spec, seed))
    return spec, net
