"""CPU oracle of the LLaMA decoder (numpy).  TEST INFRASTRUCTURE ONLY.

Restates what LiteNN's lowered graphs compute, on dequantized fp32 weights:
  decoder block   tools/gguf/LLaMABuilder.cpp:502-557 (prefill), :568-668 (decode, explicit KV)
  RMSNorm         src/LiteNN/ComputePrimitives.h:795-821 (statistics in double)
  RoPE            src/LiteNN/Layer/RoPE.h:22-114 (interleaved pairs, tables in double -> fp32)
  attention       src/LiteNN/Layer/FlashAttnExt.h:100-229 + Layer/CausalMask.h:15-33
                  (scale 1/sqrt(hd), additive -1e9 mask, max-shifted softmax, probs.V)
  SwiGLU          src/LiteNN/Layer/SwiGLU.h:54-64, Layer/Activation.h:20-33,52-59
  logits          LLaMABuilder.cpp:719-733 (final norm, output linear)
with the rounding points the benchmark configurations add on top of the reference and
that the GPU path uses: the K/V cache is fp16; in PREFILL the activations entering a
linear and the dequantized weights are rounded to bf16 (the tensor-core GEMM path), in
DECODE both stay fp32.  Accumulations are done in float64 here.
"""
from __future__ import annotations

import numpy as np

import oracle
from litenn_b200 import llama as ll
from litenn_b200 import synth


def _bf16(a):
    return oracle.fp32_to_bf16_round(np.asarray(a, dtype=np.float32))


def _fp16(a):
    return np.asarray(a, dtype=np.float32).astype(np.float16).astype(np.float32)


def _rmsnorm(x, w, eps):
    x64 = x.astype(np.float64)
    denom = np.sqrt((x64 * x64).mean(axis=-1, keepdims=True) + eps)
    return ((x64 / denom).astype(np.float32) * w).astype(np.float32)


def _silu(x):
    x = x.astype(np.float32)
    return (x / (np.float32(1.0) + np.exp(-x))).astype(np.float32)


class LlamaOracle:
    def __init__(self, spec: ll.LlamaSpec, seed: int = 0):
        self.spec = spec
        s = spec
        self.layers = []
        for layer in range(s.n_layers):
            p = ll.tensor_payloads(s, layer, seed)
            d, hd = s.d_model, s.head_dim
            w = {
                "q": oracle.dequant(s.linear_fmt, p["attn_q"], s.n_heads * hd, d),
                "k": oracle.dequant(s.linear_fmt, p["attn_k"], s.n_kv_heads * hd, d),
                "v": oracle.dequant(s.linear_fmt, p["attn_v"], s.n_kv_heads * hd, d),
                "o": oracle.dequant(s.linear_fmt, p["attn_output"], d, s.n_heads * hd),
                "gate": oracle.dequant(s.linear_fmt, p["ffn_gate"], s.ffn, d),
                "up": oracle.dequant(s.linear_fmt, p["ffn_up"], s.ffn, d),
                "down": oracle.dequant(s.dfmt, p["ffn_down"], d, s.ffn),
            }
            self.layers.append(w)
        self.embd = oracle.dequant(s.embd_fmt, synth.make_weight(s.embd_fmt, s.vocab, s.d_model, seed=seed,
                                                                 name="token_embd.weight"), s.vocab, s.d_model)
        self.head = oracle.dequant(s.embd_fmt, synth.make_weight(s.embd_fmt, s.vocab, s.d_model, seed=seed,
                                                                 name="output.weight"), s.vocab, s.d_model)
        self.norm_w = np.ones(s.d_model, dtype=np.float32)
        half = s.head_dim // 2
        pos = np.arange(s.max_seq, dtype=np.float64)[:, None]
        inv = np.power(float(s.rope_theta), -2.0 * np.arange(half, dtype=np.float64) / float(s.head_dim))[None, :]
        self.cos = np.cos(pos * inv).astype(np.float32)
        self.sin = np.sin(pos * inv).astype(np.float32)
        self.k_cache = [np.zeros((s.n_kv_heads, s.max_seq, s.head_dim), np.float32) for _ in range(s.n_layers)]
        self.v_cache = [np.zeros((s.n_kv_heads, s.max_seq, s.head_dim), np.float32) for _ in range(s.n_layers)]
        self.pos = 0
        self.last_logits = None

    # linear with the rounding of the path in use
    @staticmethod
    def _linear(x, w, prefill):
        if prefill:
            x, w = _bf16(x), _bf16(w)
        return (x.astype(np.float64) @ w.astype(np.float64).T).astype(np.float32)

    def _rope(self, x, n_heads, positions):
        s = self.spec
        x = x.reshape(len(positions), n_heads, s.head_dim // 2, 2).astype(np.float32)
        c = self.cos[positions][:, None, :]
        sn = self.sin[positions][:, None, :]
        a, b = x[..., 0], x[..., 1]
        ra = (a * c).astype(np.float32) - (b * sn).astype(np.float32)
        rb = (a * sn).astype(np.float32) + (b * c).astype(np.float32)
        return np.stack([ra, rb], axis=-1).reshape(len(positions), n_heads * s.head_dim).astype(np.float32)

    def _forward(self, tokens, prefill):
        s = self.spec
        m = len(tokens)
        positions = np.arange(self.pos, self.pos + m)
        h = self.embd[np.asarray(tokens)].astype(np.float32)
        group = s.n_heads // s.n_kv_heads
        scale = np.float32(1.0 / np.sqrt(s.head_dim))
        for l, w in enumerate(self.layers):
            xn = _rmsnorm(h, self.norm_w, s.rms_eps)
            q = self._rope(self._linear(xn, w["q"], prefill), s.n_heads, positions)
            k = self._rope(self._linear(xn, w["k"], prefill), s.n_kv_heads, positions)
            v = self._linear(xn, w["v"], prefill)
            kc, vc = self.k_cache[l], self.v_cache[l]
            kc[:, positions, :] = _fp16(k).reshape(m, s.n_kv_heads, s.head_dim).transpose(1, 0, 2)
            vc[:, positions, :] = _fp16(v).reshape(m, s.n_kv_heads, s.head_dim).transpose(1, 0, 2)
            ctx = np.zeros((m, s.n_heads * s.head_dim), np.float32)
            n_keys = self.pos + m
            for hh in range(s.n_heads):
                qh = q[:, hh * s.head_dim:(hh + 1) * s.head_dim].astype(np.float64)
                kh = kc[hh // group, :n_keys].astype(np.float64)
                vh = vc[hh // group, :n_keys].astype(np.float64)
                sc = (qh @ kh.T) * float(scale)
                mask = np.arange(n_keys)[None, :] > positions[:, None]
                sc = sc + np.where(mask, -1.0e9, 0.0)
                sc = sc - sc.max(axis=1, keepdims=True)
                p = np.exp(sc)
                p = p / p.sum(axis=1, keepdims=True)
                ctx[:, hh * s.head_dim:(hh + 1) * s.head_dim] = (p @ vh).astype(np.float32)
            h = (h + self._linear(ctx, w["o"], prefill)).astype(np.float32)
            xn = _rmsnorm(h, self.norm_w, s.rms_eps)
            act = (_silu(self._linear(xn, w["gate"], prefill)) * self._linear(xn, w["up"], prefill)).astype(np.float32)
            h = (h + self._linear(act, w["down"], prefill)).astype(np.float32)
        self.pos += m
        last = _rmsnorm(h[-1:], self.norm_w, s.rms_eps)
        self.last_logits = self._linear(last, self.head, False)[0]  # the head runs on the decode (fp32) path
        return int(np.argmax(self.last_logits))

    def prefill(self, tokens):
        return self._forward(list(tokens), True)

    def decode_step(self, token):
        return self._forward([int(token)], False)

    def top2_gap(self):
        t = np.sort(self.last_logits)[-2:]
        return float(t[1] - t[0]), float(np.abs(self.last_logits).max())
