"""Model families assembled from the add-on layers: GPT-2, GPT-J and Llama shaped decoders, their training program
(`DecoderTrainer`) and the int4 tensor-parallel decoding program (`DecoderGenerator`)."""
from .decoder import DecoderBlock, DecoderConfig, DecoderEmbedding, DecoderHead

__all__ = ["DecoderConfig", "DecoderBlock", "DecoderEmbedding", "DecoderHead"]
