"""Host-side assembly of a LLaMA decoder on top of the C ABI (include/litenn_llama.h).

Builds the random-init models of the benchmark configurations from seeded synthetic GGUF
payloads (tensor names as in tools/gguf/LLaMABuilder.cpp:473-497: ``blk.<i>.attn_q.weight``
...), shards them for tensor parallelism and hands the packed weights to the decoder.
Nothing here computes: it only moves bytes and calls the library.
"""
from __future__ import annotations

import ctypes
import dataclasses

import numpy as np

from . import capi, synth


@dataclasses.dataclass
class LlamaSpec:
    n_layers: int
    d_model: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    ffn: int
    vocab: int
    linear_fmt: int = synth.Q4_0      # attn_q/k/v/output, ffn_gate/up
    down_fmt: int | None = None       # ffn_down (defaults to linear_fmt)
    embd_fmt: int = synth.Q6_K        # token_embd and output
    rms_eps: float = 1e-6
    rope_theta: float = 10000.0
    max_seq: int = 640
    max_prefill: int = 512
    rope_dim: int | None = None       # rope.dimension_count (defaults to head_dim)
    unit_norms: bool = True           # RMSNorm weights all one (the benchmark configurations) or ~ N(1, 0.1)
    tied_output: bool = False         # no output.weight tensor: the logits reuse token_embd

    @property
    def rdim(self) -> int:
        return self.head_dim if self.rope_dim is None else self.rope_dim

    @property
    def dfmt(self) -> int:
        return self.linear_fmt if self.down_fmt is None else self.down_fmt


SPEC_7B = LlamaSpec(32, 4096, 32, 32, 128, 11008, 32000, synth.Q4_0, None, synth.Q6_K, max_seq=640, max_prefill=512)
SPEC_70B = LlamaSpec(80, 8192, 64, 8, 128, 28672, 128256, synth.Q4_K, synth.Q6_K, synth.Q6_K, max_seq=1280,
                     max_prefill=1024)


def tensor_payloads(spec: LlamaSpec, layer: int, seed: int = 0) -> dict[str, np.ndarray]:
    """Raw ggml payloads of one decoder block, keyed by GGUF tensor suffix."""
    d, hd = spec.d_model, spec.head_dim
    shapes = {
        "attn_q": (spec.n_heads * hd, d, spec.linear_fmt), "attn_k": (spec.n_kv_heads * hd, d, spec.linear_fmt),
        "attn_v": (spec.n_kv_heads * hd, d, spec.linear_fmt), "attn_output": (d, spec.n_heads * hd, spec.linear_fmt),
        "ffn_gate": (spec.ffn, d, spec.linear_fmt), "ffn_up": (spec.ffn, d, spec.linear_fmt),
        "ffn_down": (d, spec.ffn, spec.dfmt),
    }
    return {k: synth.make_weight(f, n, kk, seed=seed, name=f"blk.{layer}.{k}.weight") for k, (n, kk, f) in shapes.items()}


def norm_weights(spec: LlamaSpec, layer: int, seed: int = 0) -> dict[str, np.ndarray]:
    """RMSNorm weights of one block (``attn_norm``, ``ffn_norm``) or, for layer < 0, ``output_norm``."""
    names = ["output_norm"] if layer < 0 else [f"blk.{layer}.attn_norm", f"blk.{layer}.ffn_norm"]
    out = {}
    for n in names:
        key = n.split(".")[-1]
        out[key] = (np.ones(spec.d_model, dtype=np.float32) if spec.unit_norms
                    else synth.make_norm_weight(spec.d_model, seed=seed, name=n + ".weight"))
    return out


def shard_ranges(spec: LlamaSpec, tp_rank: int, tp_size: int) -> dict[str, tuple[str, int, int]]:
    """Which slice of every tensor a rank owns: ("rows" | "cols", begin, end).

    Megatron-style: attn_q/k/v and ffn_gate/up and output by output rows (whole heads),
    attn_output and ffn_down by input columns, which must fall on block boundaries."""
    if spec.n_heads % tp_size or spec.n_kv_heads % tp_size or spec.ffn % tp_size or spec.vocab % tp_size:
        raise ValueError("heads, kv heads, ffn width and vocabulary must divide over the ranks")
    hd, r = spec.head_dim, tp_rank
    hl, kvl, ffl, vl = spec.n_heads // tp_size, spec.n_kv_heads // tp_size, spec.ffn // tp_size, spec.vocab // tp_size
    if (hl * hd) % synth.BLOCK_ELEMS[spec.linear_fmt] or ffl % synth.BLOCK_ELEMS[spec.dfmt]:
        raise ValueError("a column shard would cut a quantization block")
    return {
        "attn_q": ("rows", r * hl * hd, (r + 1) * hl * hd),
        "attn_k": ("rows", r * kvl * hd, (r + 1) * kvl * hd),
        "attn_v": ("rows", r * kvl * hd, (r + 1) * kvl * hd),
        "attn_output": ("cols", r * hl * hd, (r + 1) * hl * hd),
        "ffn_gate": ("rows", r * ffl, (r + 1) * ffl),
        "ffn_up": ("rows", r * ffl, (r + 1) * ffl),
        "ffn_down": ("cols", r * ffl, (r + 1) * ffl),
        "output": ("rows", r * vl, (r + 1) * vl),
    }


def _rows(payload: np.ndarray, fmt: int, k: int, r0: int, r1: int) -> np.ndarray:
    rb = k // synth.BLOCK_ELEMS[fmt] * synth.BLOCK_BYTES[fmt]
    return payload[r0 * rb:r1 * rb]


class LlamaModel:
    """A decoder resident on one GPU (one tensor-parallel rank)."""

    def __init__(self, spec: LlamaSpec, device: int = 0, tp_rank: int = 0, tp_size: int = 1, stream: int = 0,
                 seed: int = 0, share_layer_payloads: bool = False):
        """``share_layer_payloads`` reuses block 0's host payloads for every block (each block still
        gets its own packed copy in HBM): the timing is unchanged and set-up is 30x faster."""
        self.spec, self.device, self.tp_rank, self.tp_size, self.stream = spec, device, tp_rank, tp_size, stream
        L = capi.load()
        cfg = capi.LlamaConfig(spec.n_layers, spec.d_model, spec.n_heads, spec.n_kv_heads, spec.head_dim, spec.ffn,
                               spec.vocab, spec.rdim, spec.max_seq, spec.max_prefill, tp_rank, tp_size,
                               spec.embd_fmt, spec.rms_eps, spec.rope_theta)
        h = ctypes.c_void_p()
        capi.check(L.qmm_llama_create(device, ctypes.byref(cfg), ctypes.byref(h)))
        self._h = h
        self._weights = []  # keep the packed weights alive
        d, hd, tp, r = spec.d_model, spec.head_dim, tp_size, tp_rank
        hl, kvl, ffl = spec.n_heads // tp, spec.n_kv_heads // tp, spec.ffn // tp
        rng = shard_ranges(spec, r, tp)
        cached = None
        for layer in range(spec.n_layers):
            if share_layer_payloads and cached is not None:
                p = cached
            else:
                p = tensor_payloads(spec, layer, seed)
                cached = p
            f = spec.linear_fmt
            qkv = np.concatenate([_rows(p[t], f, d, rng[t][1], rng[t][2]) for t in ("attn_q", "attn_k", "attn_v")])
            # gate and up rows alternate in groups of 8, so that one 16-row tile holds both halves of 8 channels
            gu = capi.interleave_gate_up(f, *(np.ascontiguousarray(_rows(p[t], f, d, rng[t][1], rng[t][2]))
                                              for t in ("ffn_gate", "ffn_up")), ffl, d)
            ws = {
                capi.LL_QKV: capi.Weight.from_host(f, qkv, (hl + 2 * kvl) * hd, d, device, stream),
                capi.LL_O: capi.Weight.from_host(f, p["attn_output"], d, spec.n_heads * hd, device, stream,
                                                 capi.SPLIT_K if tp > 1 else capi.SPLIT_NONE, r, tp),
                capi.LL_GU: capi.Weight.from_host(f, gu, 2 * ffl, d, device, stream),
                capi.LL_DOWN: capi.Weight.from_host(spec.dfmt, p["ffn_down"], d, spec.ffn, device, stream,
                                                    capi.SPLIT_K if tp > 1 else capi.SPLIT_NONE, r, tp),
            }
            for which, w in ws.items():
                capi.check(L.qmm_llama_set_weight(self._h, layer, which, w.handle))
                self._weights.append(w)
            nw = norm_weights(spec, layer, seed)
            for which, key in ((capi.LL_ATTN_NORM, "attn_norm"), (capi.LL_FFN_NORM, "ffn_norm")):
                capi.check(L.qmm_llama_set_norm(self._h, layer, which, ctypes.c_void_p(nw[key].ctypes.data)))
        fw = norm_weights(spec, -1, seed)["output_norm"]
        capi.check(L.qmm_llama_set_norm(self._h, -1, capi.LL_FINAL_NORM, ctypes.c_void_p(fw.ctypes.data)))
        embd = synth.make_weight(spec.embd_fmt, spec.vocab, d, seed=seed, name="token_embd.weight")
        capi.check(L.qmm_llama_set_embedding(self._h, ctypes.c_void_p(embd.ctypes.data), embd.nbytes))
        if spec.tied_output:
            capi.check(L.qmm_llama_tie_output(self._h, ctypes.c_void_p(embd.ctypes.data), embd.nbytes,
                                              ctypes.c_void_p(stream)))
        else:
            out = synth.make_weight(spec.embd_fmt, spec.vocab, d, seed=seed, name="output.weight")
            head = capi.Weight.from_host(spec.embd_fmt, out, spec.vocab, d, device, stream,
                                         capi.SPLIT_N if tp > 1 else capi.SPLIT_NONE, r, tp)
            capi.check(L.qmm_llama_set_weight(self._h, -1, capi.LL_HEAD, head.handle))
            self._weights.append(head)

    def tp_init(self, nccl_path: str, unique_id: bytes) -> None:
        capi.check(capi.load().qmm_llama_tp_init(self._h, nccl_path.encode(), unique_id))

    def tp_export(self) -> bytes:
        """This rank's 128-byte exchange record (qmm_llama_tp_export)."""
        buf = ctypes.create_string_buffer(128)
        capi.check(capi.load().qmm_llama_tp_export(self._h, buf))
        return buf.raw

    def tp_import(self, records: list[bytes]) -> None:
        """Records of all ranks in rank order (qmm_llama_tp_import): decode then sums over peer memory."""
        if len(records) != self.tp_size or any(len(r) != 128 for r in records):
            raise ValueError("one 128-byte record per rank is required")
        capi.check(capi.load().qmm_llama_tp_import(self._h, b"".join(records), ctypes.c_void_p(self.stream)))

    def tp_loopback(self) -> None:
        """Test hook (qmm_llama_tp_loopback): peers that never answer, on one GPU."""
        capi.check(capi.load().qmm_llama_tp_loopback(self._h))

    def set_wait_limit(self, polls: int) -> None:
        capi.check(capi.load().qmm_llama_set_wait_limit(self._h, int(polls)))

    def set_collective_timeout(self, milliseconds: int) -> None:
        capi.check(capi.load().qmm_llama_set_collective_timeout(self._h, int(milliseconds)))

    def generated(self, first: int, count: int) -> np.ndarray:
        """Generated tokens first .. first+count-1 since the last reset (synchronizes)."""
        out = np.empty(count, dtype=np.int32)
        capi.check(capi.load().qmm_llama_generated_tokens(self._h, first, count, ctypes.c_void_p(out.ctypes.data),
                                                          ctypes.c_void_p(self.stream)))
        return out

    def has_graph(self) -> bool:
        return bool(capi.load().qmm_llama_has_graph(self._h))

    # ---- batched decode: independent sequences that share the weights --------------------------------
    def batch_create(self, batch: int, max_steps: int) -> None:
        capi.check(capi.load().qmm_llama_batch_create(self._h, int(batch), int(max_steps)))
        self.batch = int(batch)

    def batch_prefill(self, seq: int, tokens: np.ndarray) -> int:
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        first = ctypes.c_int32()
        capi.check(capi.load().qmm_llama_batch_prefill(self._h, int(seq), ctypes.c_void_p(tokens.ctypes.data), len(tokens),
                                                       ctypes.byref(first), ctypes.c_void_p(self.stream)))
        return int(first.value)

    def batch_decode(self, steps: int) -> np.ndarray:
        """tokens[step, sequence] of the next `steps` steps."""
        out = np.empty((steps, self.batch), dtype=np.int32)
        capi.check(capi.load().qmm_llama_batch_decode(self._h, int(steps), ctypes.c_void_p(out.ctypes.data),
                                                      ctypes.c_void_p(self.stream)))
        return out

    def batch_decode_enqueue(self, steps: int) -> None:
        capi.check(capi.load().qmm_llama_batch_decode_enqueue(self._h, int(steps), ctypes.c_void_p(self.stream)))

    def batch_generated(self, first_step: int, steps: int) -> np.ndarray:
        out = np.empty((steps, self.batch), dtype=np.int32)
        capi.check(capi.load().qmm_llama_batch_generated_tokens(self._h, int(first_step), int(steps),
                                                                ctypes.c_void_p(out.ctypes.data),
                                                                ctypes.c_void_p(self.stream)))
        return out

    def reset(self) -> None:
        capi.check(capi.load().qmm_llama_reset(self._h, ctypes.c_void_p(self.stream)))

    def prefill(self, tokens: np.ndarray) -> int:
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        first = ctypes.c_int32()
        capi.check(capi.load().qmm_llama_prefill(self._h, ctypes.c_void_p(tokens.ctypes.data), len(tokens),
                                                 ctypes.byref(first), ctypes.c_void_p(self.stream)))
        return int(first.value)

    def decode(self, steps: int) -> np.ndarray:
        out = np.empty(steps, dtype=np.int32)
        capi.check(capi.load().qmm_llama_decode(self._h, steps, ctypes.c_void_p(out.ctypes.data),
                                                ctypes.c_void_p(self.stream)))
        return out

    def decode_enqueue(self, steps: int) -> None:
        capi.check(capi.load().qmm_llama_decode_enqueue(self._h, steps, ctypes.c_void_p(self.stream)))

    def step_host(self, token: int) -> int:
        out = ctypes.c_int32()
        capi.check(capi.load().qmm_llama_step_host(self._h, int(token), ctypes.byref(out), ctypes.c_void_p(self.stream)))
        return int(out.value)

    def last_logits(self) -> np.ndarray:
        out = np.empty(self.spec.vocab // self.tp_size, dtype=np.float32)
        capi.check(capi.load().qmm_llama_last_logits(self._h, ctypes.c_void_p(out.ctypes.data),
                                                     ctypes.c_void_p(self.stream)))
        return out

    def close(self) -> None:
        if self._h:
            h, self._h = self._h, ctypes.c_void_p()
            capi.check(capi.load().qmm_llama_destroy(h))
            self._weights.clear()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def nccl_unique_id(nccl_path: str) -> bytes:
    buf = ctypes.create_string_buffer(128)
    capi.check(capi.load().qmm_llama_tp_unique_id(nccl_path.encode(), buf))
    return buf.raw


def find_nccl_library() -> str:
    """The NCCL shared library bundled with PyTorch (nvidia-nccl wheel), else the system one."""
    import glob
    import os
    import sys
    for base in sys.path:
        hits = glob.glob(os.path.join(base, "nvidia", "nccl", "lib", "libnccl.so*"))
        if hits:
            return sorted(hits)[0]
    return "libnccl.so.2"
