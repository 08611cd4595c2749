"""CPU oracle of the LLaMA decoder (numpy).  TEST INFRASTRUCTURE ONLY.

Restates what LiteNN's lowered graphs compute, on dequantized fp32 weights:
  decoder block   tools/gguf/LLaMABuilder.cpp:502-557 (prefill), :568-668 (decode, explicit KV)
  RMSNorm         src/LiteNN/ComputePrimitives.h:755-816 (mean of squares, division, scale: all in
                  double; ONE cast to the tensor's type at the end)
  RoPE            src/LiteNN/Layer/RoPE.h:22-114 (interleaved pairs, tables in double -> fp32, products
                  and sums as separate fp32 graph nodes); only the first rope.dimension_count
                  elements of a head rotate, with frequencies over that count
                  (LLaMABuilder.cpp:311-348)
  attention       src/LiteNN/Layer/FlashAttnExt.h:100-229 + Layer/CausalMask.h:15-33
                  (scale 1/sqrt(hd), additive -1e9 mask, max-shifted softmax, probs.V)
  SwiGLU          src/LiteNN/Layer/SwiGLU.h:54-64, Layer/Activation.h:20-33,52-59
  logits          LLaMABuilder.cpp:719-733 (final norm, output linear; token_embd when there is no
                  output.weight)
The building blocks are module-level functions so that tests/test_llama_oracle_pins.py can hold
them against the known answers of the reference's own layer tests (tests/LayerTest.cpp).

Rounding points that the benchmark configurations add on top of the reference and that the GPU
path uses: the K/V cache is fp16; in PREFILL the activations entering a linear and the
dequantized weights are rounded to bf16 (the tensor-core GEMM path), in DECODE both stay fp32.
Accumulations are done in float64 here.
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


def rmsnorm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis; double throughout, one cast (w may be None)."""
    x64 = np.asarray(x, dtype=np.float32).astype(np.float64)
    denom = np.sqrt((x64 * x64).mean(axis=-1, keepdims=True) + float(eps))
    out = x64 / denom
    if w is not None:
        out = out * np.asarray(w, dtype=np.float32).astype(np.float64)
    return out.astype(np.float32)


def rope_tables(n_pos, rope_dim, base, position_offset=0, frequency_scale=1.0):
    """cos/sin [n_pos, rope_dim/2] as the reference builds them: in double, cast to fp32."""
    half = rope_dim // 2
    pos = (np.arange(n_pos, dtype=np.float64) + float(position_offset))[:, None]
    inv = np.power(float(base), -2.0 * np.arange(half, dtype=np.float64) / float(half * 2))[None, :]
    ang = pos * inv * float(frequency_scale)
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def rope(x, cos, sin):
    """Rotate interleaved pairs of x [rows, features] with per-row tables [rows, features/2]."""
    x = np.asarray(x, dtype=np.float32)
    rows, feat = x.shape
    p = x.reshape(rows, feat // 2, 2)
    a, b = p[..., 0], p[..., 1]
    ra = (a * cos).astype(np.float32) - (b * sin).astype(np.float32)
    rb = (a * sin).astype(np.float32) + (b * cos).astype(np.float32)
    return np.stack([ra, rb], axis=-1).reshape(rows, feat).astype(np.float32)


def silu(x):
    x = np.asarray(x, dtype=np.float32)
    sig = (np.float32(1.0) / (np.float32(1.0) + np.exp(-x))).astype(np.float32)
    return (x * sig).astype(np.float32)


def swiglu(x, w_gate, w_up, w_down):
    """down(silu(gate(x)) * up(x)) with weights [in, out] as Layer::CreateSwiGLUMLP takes them."""
    x = np.asarray(x, dtype=np.float64)
    g = (x @ np.asarray(w_gate, dtype=np.float64)).astype(np.float32)
    u = (x @ np.asarray(w_up, dtype=np.float64)).astype(np.float32)
    act = (silu(g) * u).astype(np.float32)
    return (act.astype(np.float64) @ np.asarray(w_down, dtype=np.float64)).astype(np.float32)


def attention(q, k, v, scale, causal=True, query_offset=0, key_offset=0):
    """softmax(q.k^T * scale + mask) . v; the causal mask adds -1e9 where key position > query position."""
    q64, k64, v64 = (np.asarray(t, dtype=np.float32).astype(np.float64) for t in (q, k, v))
    sc = (q64 @ k64.T) * float(scale)
    if causal:
        qpos = np.arange(q64.shape[0])[:, None] + query_offset
        kpos = np.arange(k64.shape[0])[None, :] + key_offset
        sc = sc + np.where(kpos > qpos, -1.0e9, 0.0)
    sc = sc - sc.max(axis=1, keepdims=True)
    p = np.exp(sc)
    p = p / p.sum(axis=1, keepdims=True)
    return (p @ v64).astype(np.float32)


def kv_append(past, new):
    return np.concatenate([np.asarray(past, dtype=np.float32), np.asarray(new, dtype=np.float32)], axis=0)


class LlamaOracle:
    def __init__(self, spec: ll.LlamaSpec, seed: int = 0, share_layer_payloads: bool = False):
        self.spec = spec
        s = spec
        self.layers = []
        self.norms = []
        for layer in range(s.n_layers):
            if share_layer_payloads and self.layers:
                self.layers.append(self.layers[0])
            else:
                p = ll.tensor_payloads(s, layer, seed)
                d, hd = s.d_model, s.head_dim
                self.layers.append({
                    "q": oracle.dequant(s.linear_fmt, p["attn_q"], s.n_heads * hd, d),
                    "k": oracle.dequant(s.linear_fmt, p["attn_k"], s.n_kv_heads * hd, d),
                    "v": oracle.dequant(s.linear_fmt, p["attn_v"], s.n_kv_heads * hd, d),
                    "o": oracle.dequant(s.linear_fmt, p["attn_output"], d, s.n_heads * hd),
                    "gate": oracle.dequant(s.linear_fmt, p["ffn_gate"], s.ffn, d),
                    "up": oracle.dequant(s.linear_fmt, p["ffn_up"], s.ffn, d),
                    "down": oracle.dequant(s.dfmt, p["ffn_down"], d, s.ffn),
                })
            self.norms.append(ll.norm_weights(s, layer, seed))
        self.final_norm = ll.norm_weights(s, -1, seed)["output_norm"]
        self.embd = oracle.dequant(s.embd_fmt, synth.make_weight(s.embd_fmt, s.vocab, s.d_model, seed=seed,
                                                                 name="token_embd.weight"), s.vocab, s.d_model)
        if s.tied_output:
            self.head = self.embd
        else:
            self.head = oracle.dequant(s.embd_fmt, synth.make_weight(s.embd_fmt, s.vocab, s.d_model, seed=seed,
                                                                     name="output.weight"), s.vocab, s.d_model)
        self.cos, self.sin = rope_tables(s.max_seq, s.rdim, s.rope_theta)
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
        # one or a few rows: the threaded C loop with double accumulation avoids a float64 copy of w
        return oracle.matmul_nk_f64(np.ascontiguousarray(x, dtype=np.float32), w).astype(np.float32)

    def _rope_heads(self, x, n_heads, positions):
        s = self.spec
        m = len(positions)
        x = np.asarray(x, dtype=np.float32).reshape(m * n_heads, s.head_dim).copy()
        cos = np.repeat(self.cos[positions], n_heads, axis=0)
        sin = np.repeat(self.sin[positions], n_heads, axis=0)
        x[:, :s.rdim] = rope(x[:, :s.rdim], cos, sin)
        return x.reshape(m, n_heads * s.head_dim)

    def _forward(self, tokens, prefill):
        s = self.spec
        m = len(tokens)
        positions = np.arange(self.pos, self.pos + m)
        h = self.embd[np.asarray(tokens)].astype(np.float32)
        group = s.n_heads // s.n_kv_heads
        scale = 1.0 / np.sqrt(s.head_dim)
        for l, w in enumerate(self.layers):
            xn = rmsnorm(h, self.norms[l]["attn_norm"], s.rms_eps)
            q = self._rope_heads(self._linear(xn, w["q"], prefill), s.n_heads, positions)
            k = self._rope_heads(self._linear(xn, w["k"], prefill), s.n_kv_heads, positions)
            v = self._linear(xn, w["v"], prefill)
            kc, vc = self.k_cache[l], self.v_cache[l]
            kc[:, positions, :] = _fp16(k).reshape(m, s.n_kv_heads, s.head_dim).transpose(1, 0, 2)
            vc[:, positions, :] = _fp16(v).reshape(m, s.n_kv_heads, s.head_dim).transpose(1, 0, 2)
            ctx = np.zeros((m, s.n_heads * s.head_dim), np.float32)
            n_keys = self.pos + m
            for hh in range(s.n_heads):
                qh = q[:, hh * s.head_dim:(hh + 1) * s.head_dim]
                ctx[:, hh * s.head_dim:(hh + 1) * s.head_dim] = attention(
                    qh, kc[hh // group, :n_keys], vc[hh // group, :n_keys], scale, True, query_offset=self.pos)
            h = (h + self._linear(ctx, w["o"], prefill)).astype(np.float32)
            xn = rmsnorm(h, self.norms[l]["ffn_norm"], s.rms_eps)
            act = (silu(self._linear(xn, w["gate"], prefill)) * self._linear(xn, w["up"], prefill)).astype(np.float32)
            h = (h + self._linear(act, w["down"], prefill)).astype(np.float32)
        self.pos += m
        last = rmsnorm(h[-1:], self.final_norm, s.rms_eps)
        self.last_logits = self._linear(last, self.head, False)[0]  # the head runs on the decode (fp32) path
        return int(np.argmax(self.last_logits))

    def prefill(self, tokens):
        return self._forward(list(tokens), True)

    def decode_step(self, token):
        return self._forward([int(token)], False)

    def top2_gap(self):
        t = np.sort(self.last_logits)[-2:]
        return float(t[1] - t[0]), float(np.abs(self.last_logits).max())
