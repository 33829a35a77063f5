"""Greedy generation with int4 weights: the traced prefill + decode program against a plain PyTorch forward pass that
uses the de-quantised weights, for tp=1 and (simulated) tp=2."""
import dataclasses

import numpy as np
import pytest
import torch

from popxl_addons_b200.models.decoder import DecoderConfig
from popxl_addons_b200.models.generator import DecoderGenerator, quantize_rows
from popxl_addons_b200.ops.rotary_pos_embed import trig_tables


def _dense_weights(cfg, seed=0):
    rs = np.random.RandomState(seed)
    hd = cfg.heads * cfg.head_dim
    w = {"wte": rs.normal(0, 0.5, (cfg.vocab_size, cfg.hidden)), "lm_head": rs.normal(0, 0.3, (cfg.vocab_size, cfg.hidden)),
         "lm_head.bias": rs.normal(0, 0.1, (cfg.vocab_size,)),
         "ln_f.weight": 1 + 0.1 * rs.normal(size=cfg.hidden), "ln_f.bias": 0.1 * rs.normal(size=cfg.hidden)}
    for i in range(cfg.layers):
        w[f"layer{i}.ln_1.weight"] = 1 + 0.1 * rs.normal(size=cfg.hidden)
        w[f"layer{i}.ln_1.bias"] = 0.1 * rs.normal(size=cfg.hidden)
        w[f"layer{i}.qkv"] = rs.normal(0, 0.2, (3 * hd, cfg.hidden))
        w[f"layer{i}.out"] = rs.normal(0, 0.2, (cfg.hidden, hd))
        w[f"layer{i}.fc_in"] = rs.normal(0, 0.2, (cfg.ffn, cfg.hidden))
        w[f"layer{i}.fc_in.bias"] = rs.normal(0, 0.1, (cfg.ffn,))
        w[f"layer{i}.fc_out"] = rs.normal(0, 0.2, (cfg.hidden, cfg.ffn))
        w[f"layer{i}.fc_out.bias"] = rs.normal(0, 0.1, (cfg.hidden,))
    return {k: v.astype(np.float32) for k, v in w.items()}


def _dequant(w, gs):
    packed, scale, zero = quantize_rows(torch.tensor(w), gs)
    p = packed.to(torch.int32) & 0xFFFF
    codes = torch.stack([(p >> 12) & 15, (p >> 8) & 15, (p >> 4) & 15, p & 15], dim=-1).float()
    codes = codes.reshape(w.shape[0], w.shape[1] // gs, gs)
    return (codes * scale + zero).reshape(w.shape)


def _rotate(x, sin, cos, rd):
    rot, rest = x[..., :rd], x[..., rd:]
    re, im = rot[..., 0::2], rot[..., 1::2]
    y = torch.stack((re * cos - im * sin, im * cos + re * sin), dim=-1).flatten(-2)
    return torch.cat((y, rest), dim=-1)


def _reference_generate(cfg, w, prompt, n_new, gs):
    """Recomputes the whole sequence for every new token (no cache)."""
    W = {k: (_dequant(v, gs) if v.ndim == 2 and k != "wte" else torch.tensor(v)) for k, v in w.items()}
    toks = torch.tensor(prompt, dtype=torch.long)
    H, D = cfg.heads, cfg.head_dim
    out = []
    for _ in range(n_new):
        B, S = toks.shape
        sin, cos = (torch.tensor(t) for t in trig_tables(S, cfg.rotary_dim))
        x = W["wte"][toks]
        for i in range(cfg.layers):
            h = torch.nn.functional.layer_norm(x, (cfg.hidden,), W[f"layer{i}.ln_1.weight"], W[f"layer{i}.ln_1.bias"],
                                               cfg.eps)
            qkv = h @ W[f"layer{i}.qkv"].T
            q, k, v = (t.reshape(B, S, H, D).permute(0, 2, 1, 3) for t in qkv.chunk(3, dim=-1))
            q, k = _rotate(q, sin, cos, cfg.rotary_dim), _rotate(k, sin, cos, cfg.rotary_dim)
            s = q @ k.transpose(-1, -2) / np.sqrt(D)
            s = s.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool), 1), float("-inf"))
            a = (torch.softmax(s, -1) @ v).permute(0, 2, 1, 3).reshape(B, S, H * D)
            o = a @ W[f"layer{i}.out"].T
            z = torch.nn.functional.gelu(h @ W[f"layer{i}.fc_in"].T + W[f"layer{i}.fc_in.bias"])
            x = x + o + z @ W[f"layer{i}.fc_out"].T + W[f"layer{i}.fc_out.bias"]
        hn = torch.nn.functional.layer_norm(x[:, -1], (cfg.hidden,), W["ln_f.weight"], W["ln_f.bias"], cfg.eps)
        logits = hn @ W["lm_head"].T + W["lm_head.bias"]
        nxt = logits.argmax(-1)
        out.append(nxt)
        toks = torch.cat([toks, nxt[:, None]], dim=1)
    return torch.stack(out, dim=1).numpy()


@pytest.mark.parametrize("tp", [1, 2])
def test_greedy_generation_matches_dense_reference(tp):
    cfg = dataclasses.replace(DecoderConfig.tiny(tp=tp, dp=1), dtype="float32", vocab_size=501)
    gs, B, P, N = 16, 3, 7, 6
    gen = DecoderGenerator(cfg, batch=B, prompt_len=P, max_new_tokens=N, group_size=gs, device="cpu", cuda_graphs=False)
    w = _dense_weights(cfg)
    gen.load_dense(w)
    prompt = np.random.RandomState(1).randint(0, cfg.vocab_size, (B, P)).astype(np.int32)
    got = gen.generate(prompt)
    want = _reference_generate(cfg, w, prompt, N, gs)
    np.testing.assert_array_equal(got, want)
    # a second call restarts from the prompt (position and caches are re-initialised by the program)
    np.testing.assert_array_equal(gen.generate(prompt), want)


def test_quantize_rows_round_trip_error_is_half_a_step():
    w = torch.randn(8, 64)
    deq = _dequant(w.numpy(), 16)
    step = (w.reshape(8, 4, 16).amax(-1) - w.reshape(8, 4, 16).amin(-1)) / 15
    err = (deq - w).reshape(8, 4, 16).abs().amax(-1)
    assert torch.all(err <= step / 2 + 1e-6)


def test_random_init_generates_in_vocab_tokens():
    cfg = DecoderConfig.tiny(tp=2, dp=1)
    gen = DecoderGenerator(cfg, batch=2, prompt_len=8, max_new_tokens=4, group_size=16, device="cpu", cuda_graphs=False)
    prompt = np.random.RandomState(0).randint(0, cfg.vocab_size, (2, 8)).astype(np.int32)
    out = gen.generate(prompt)
    assert out.shape == (2, 4) and out.min() >= 0 and out.max() < cfg.vocab_size
