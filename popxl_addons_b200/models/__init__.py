"""Model families assembled from the add-on layers: GPT-2, GPT-J and Llama shaped decoders, their training program
(`DecoderTrainer`) and the int4 tensor-parallel decoding program (`DecoderGenerator`)."""
from .decoder import DecoderBlock, DecoderConfig, DecoderEmbedding, DecoderHead

__all__ = ["DecoderConfig", "DecoderBlock", "DecoderEmbedding", "DecoderHead", "DecoderTrainer", "PipelineTrainer",
           "DecoderGenerator"]

_LAZY = {"DecoderTrainer": "trainer", "PipelineTrainer": "pipeline_trainer", "DecoderGenerator": "generator"}


def __getattr__(name):
    # the programs import the transforms and the session: loaded on first use
    if name in _LAZY:
        import importlib

        return getattr(importlib.import_module(f"{__name__}.{_LAZY[name]}"), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
