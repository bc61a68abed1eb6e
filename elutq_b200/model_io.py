"""Whole-model export directories of the reference (one decoder-only Llama-shaped model).

Layout written by the reference's quantizer driver (GPTQ/llama.py:286-343, GPTQ/HLQ.py:71-73)
and read by its C++ runtime (C++/examples/models/llama.cpp:59-115):

    <dir>/embed_tokens.bin                           fp16 [vocab][hidden]
    <dir>/final_rmsnorm_weight.bin                   fp16 [hidden]
    <dir>/lm_head/lm_head/                           one linear directory (w4g128, HLQ.py:76-78), or
    <dir>/lm_head.bin                                fp16 [vocab][hidden], or
    <dir>/shared_embed_lm_head.bin                   tied embedding / lm_head, fp16 [vocab][hidden]
    <dir>/<L>/input_layernorm_weight.bin             fp16 [hidden]
    <dir>/<L>/post_attention_layernorm_weight.bin    fp16 [hidden]
    <dir>/<L>/self_attn.{q,k,v,o}_proj/              linear directories (format.read_export_dir)
    <dir>/<L>/mlp.{gate,up,down}_proj/

Everything here is host-side numpy; `decoder.TPDecoder.from_export` turns a ModelExport into
device weights (sharded over the tensor-parallel ranks).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Union

import numpy as np

from .format import ExportedLinear, read_export_dir, write_export_dir

PROJ_DIRS = {
    "q": "self_attn.q_proj", "k": "self_attn.k_proj", "v": "self_attn.v_proj", "o": "self_attn.o_proj",
    "gate": "mlp.gate_proj", "up": "mlp.up_proj", "down": "mlp.down_proj",
}


@dataclass
class LayerExport:
    linears: Dict[str, ExportedLinear]      # keys of PROJ_DIRS
    ln1: np.ndarray                         # input_layernorm weight, fp16 [hidden]
    ln2: np.ndarray                         # post_attention_layernorm weight, fp16 [hidden]


@dataclass
class ModelExport:
    embed: np.ndarray                       # fp16 [vocab][hidden]
    final_norm: np.ndarray                  # fp16 [hidden]
    lm_head: Union[ExportedLinear, np.ndarray]   # quantized linear, or fp16 [vocab][hidden]
    layers: List[LayerExport] = field(default_factory=list)
    tied: bool = False                      # lm_head is the embedding (shared_embed_lm_head.bin)

    @property
    def hidden(self) -> int:
        return int(self.final_norm.shape[0])

    @property
    def vocab(self) -> int:
        return int(self.embed.shape[0])

    @property
    def ffn(self) -> int:
        return int(self.layers[0].linears["gate"].out_channel)


def _f16(path: str, count: Optional[int] = None) -> np.ndarray:
    if not os.path.exists(path):
        raise RuntimeError(f"File is not exists: {path}")
    a = np.fromfile(path, dtype=np.float16)
    if count is not None and a.size != count:
        raise ValueError(f"{path} holds {a.size} values, expected {count}")
    return a


def write_model_export(path: str, model: ModelExport, write_groupsize: bool = False) -> None:
    """Write a model directory with the reference exporter's file names."""
    os.makedirs(path, exist_ok=True)
    emb = np.ascontiguousarray(model.embed, dtype=np.float16)
    if model.tied:
        emb.tofile(os.path.join(path, "shared_embed_lm_head.bin"))
    else:
        emb.tofile(os.path.join(path, "embed_tokens.bin"))
        if isinstance(model.lm_head, ExportedLinear):
            write_export_dir(os.path.join(path, "lm_head", "lm_head"), model.lm_head, write_groupsize)
        else:
            np.ascontiguousarray(model.lm_head, dtype=np.float16).tofile(os.path.join(path, "lm_head.bin"))
    np.ascontiguousarray(model.final_norm, dtype=np.float16).tofile(os.path.join(path, "final_rmsnorm_weight.bin"))
    for li, layer in enumerate(model.layers):
        ldir = os.path.join(path, str(li))
        os.makedirs(ldir, exist_ok=True)
        np.ascontiguousarray(layer.ln1, dtype=np.float16).tofile(os.path.join(ldir, "input_layernorm_weight.bin"))
        np.ascontiguousarray(layer.ln2, dtype=np.float16).tofile(
            os.path.join(ldir, "post_attention_layernorm_weight.bin"))
        for key, sub in PROJ_DIRS.items():
            write_export_dir(os.path.join(ldir, sub), layer.linears[key], write_groupsize)


def read_model_export(path: str, num_layers: Optional[int] = None) -> ModelExport:
    """Read a model directory (llama.cpp:59-115).  The layer count is taken from the numbered
    sub-directories unless given; hidden size from final_rmsnorm_weight.bin; vocabulary from the
    embedding's size.  A quantized lm_head directory wins over lm_head.bin, as in the reference
    (llama.cpp:69-80)."""
    final_norm = _f16(os.path.join(path, "final_rmsnorm_weight.bin"))
    hidden = final_norm.size
    if hidden == 0:
        raise ValueError("final_rmsnorm_weight.bin is empty")
    tied_path = os.path.join(path, "shared_embed_lm_head.bin")
    tied = os.path.exists(tied_path) and not os.path.exists(os.path.join(path, "embed_tokens.bin"))
    emb = _f16(tied_path if tied else os.path.join(path, "embed_tokens.bin"))
    if emb.size % hidden:
        raise ValueError("the embedding's size is not a multiple of the hidden size")
    emb = emb.reshape(-1, hidden)
    lm_dir = os.path.join(path, "lm_head", "lm_head")
    if os.path.isdir(lm_dir):
        lm_head: Union[ExportedLinear, np.ndarray] = read_export_dir(lm_dir)
        if lm_head.in_channel != hidden or lm_head.out_channel != emb.shape[0]:
            raise ValueError("lm_head does not match the embedding's shape")
        tied = False
    elif tied:
        lm_head = emb
    else:
        lm_head = _f16(os.path.join(path, "lm_head.bin"), emb.size).reshape(emb.shape)
    if num_layers is None:
        num_layers = 0
        while os.path.isdir(os.path.join(path, str(num_layers))):
            num_layers += 1
    if num_layers <= 0:
        raise ValueError(f"no layer directories under {path}")
    layers = []
    for li in range(num_layers):
        ldir = os.path.join(path, str(li))
        lin = {key: read_export_dir(os.path.join(ldir, sub)) for key, sub in PROJ_DIRS.items()}
        for key in ("q", "k", "v", "gate", "up"):
            if lin[key].in_channel != hidden:
                raise ValueError(f"layer {li} {key}: {lin[key].in_channel} input channels, hidden size is {hidden}")
        for key in ("o", "down"):
            if lin[key].out_channel != hidden:
                raise ValueError(f"layer {li} {key}: {lin[key].out_channel} output channels, hidden size is {hidden}")
        if lin["gate"].out_channel != lin["up"].out_channel or lin["down"].in_channel != lin["up"].out_channel:
            raise ValueError(f"layer {li}: gate/up/down shapes do not fit")
        layers.append(LayerExport(lin, _f16(os.path.join(ldir, "input_layernorm_weight.bin"), hidden),
                                  _f16(os.path.join(ldir, "post_attention_layernorm_weight.bin"), hidden)))
    return ModelExport(emb, final_norm, lm_head, layers, tied)
