"""GPT-J shapes (parallel attention / feed-forward residual, rotary on the first 64 features of each 256-wide head)."""
from .decoder import DecoderConfig


class GPTJConfig(DecoderConfig):
    @classmethod
    def gptj_6b(cls, **kw):
        return DecoderConfig.gptj_6b(**kw)

    @classmethod
    def tiny(cls, **kw):
        # large enough for the tensor-core and vectorised kernels to take every operand (multiples of 8, >= one tile)
        base = dict(layers=2, hidden=256, heads=4, head_dim=64, rotary_dim=32, ffn=512, vocab_size=1024, seq_len=128)
        base.update(kw)
        return DecoderConfig(family="gptj", **base)
