"""Model registry: config.json's "architecture" names the class that serves a model folder.

    model = load_model("/path/to/model", dtype="bfloat16", max_tokens=..., max_seqs=...)

Folder layout: config.json (+ model.safetensors for the config-driven stacks, or the raw .bin weight tree of the
reference for the two fixed decoders, named by config "weights", default the folder itself)."""
import json
import os

MODEL_REGISTRY = {}


def register_model(architecture, loader):
    """loader(path, config, dtype, **engine_kw) -> model"""
    MODEL_REGISTRY[architecture] = loader


def read_config(path):
    with open(os.path.join(path, "config.json")) as f:
        return json.load(f)


def load_model(path, dtype="bfloat16", **kw):
    config = read_config(path)
    arch = config.get("architecture")
    if arch not in MODEL_REGISTRY:
        raise ValueError(f"unknown architecture {arch!r}; registered: {sorted(MODEL_REGISTRY)}")
    return MODEL_REGISTRY[arch](path, config, dtype, **kw)


def _load_hybrid(path, config, dtype, **kw):
    from .hybrid import HybridDecoder
    from .safetensors_io import load_file
    return HybridDecoder(config, load_file(os.path.join(path, "model.safetensors")), dtype, **kw)


def _fixed_decoder(cls_name):
    def load(path, config, dtype, **kw):
        from . import decoders
        cls = getattr(decoders, cls_name)
        m = cls(*(int(config[k]) for k in ("num_layers", "num_heads", "head_dim", "hidden_dim", "vocab_size",
                                           "max_seq_len")), batch_size=int(kw.get("max_seqs", 1)))
        wdir = os.path.join(path, config.get("weights", "."))
        (m.load_quantized_weights if cls_name == "INT8Decoder" else m.load_weights)(wdir)
        return m
    return load


for _arch in ("Megusun", "Domilix", "Dubarax", "Gunulorn"):
    register_model(_arch, _load_hybrid)
register_model("CUDADecoder", _fixed_decoder("CUDADecoder"))
register_model("INT8Decoder", _fixed_decoder("INT8Decoder"))
