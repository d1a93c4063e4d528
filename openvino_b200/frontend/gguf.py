"""GGUF frontend: reads a GGUF file (llama.cpp's container) and *builds* the decoder graph from its metadata.

GGUF stores hyper-parameters as key/value metadata and weights as named tensors in ggml types. Nothing in the file
describes a graph, so - like the reference's GGUF frontend (src/frontends/gguf/src/: gguf_reader, quant/ dequantisers,
builder/arch/decoder_builder.cpp, builder/blocks/attention.cpp, ffn.cpp) - the frontend recreates the canonical
stateful decoder topology for the architecture named in ``general.architecture`` and fills it with the tensors.

Supported: architecture ``llama`` (and layouts identical to it: mistral, qwen2 without biases); tensor types F32, F16,
BF16, Q8_0, Q4_0, Q4_1 (dequantised to float on load; pass ``compress="int4"``/``"int8"`` to re-compress group-wise for
the device kernels). llama.cpp permutes the rows of the query/key projections for its interleaved rotary embedding;
they are permuted back to the half-rotate convention that the graph uses.
"""
from __future__ import annotations

import struct
from typing import Any, BinaryIO, Dict, Optional, Tuple

import numpy as np

GGUF_MAGIC = b"GGUF"
_SCALARS = {0: ("<B", 1), 1: ("<b", 1), 2: ("<H", 2), 3: ("<h", 2), 4: ("<I", 4), 5: ("<i", 4), 6: ("<f", 4), 7: ("<?", 1), 10: ("<Q", 8),
            11: ("<q", 8), 12: ("<d", 8)}
T_STRING, T_ARRAY = 8, 9
# ggml tensor types: (block elements, block bytes)
GGML = {0: ("F32", 1, 4), 1: ("F16", 1, 2), 2: ("Q4_0", 32, 18), 3: ("Q4_1", 32, 20), 8: ("Q8_0", 32, 34), 30: ("BF16", 1, 2)}


class GgufError(RuntimeError):
    pass


def _read_str(f: BinaryIO) -> str:
    (n,) = struct.unpack("<Q", f.read(8))
    return f.read(n).decode("utf-8", errors="replace")


def _read_value(f: BinaryIO, t: int):
    if t in _SCALARS:
        fmt, n = _SCALARS[t]
        return struct.unpack(fmt, f.read(n))[0]
    if t == T_STRING:
        return _read_str(f)
    if t == T_ARRAY:
        (et,) = struct.unpack("<I", f.read(4))
        (n,) = struct.unpack("<Q", f.read(8))
        if et in _SCALARS and et != 7:
            fmt, size = _SCALARS[et]
            return np.frombuffer(f.read(size * n), dtype=np.dtype(fmt[1:]).newbyteorder("<")).tolist() if n < 4096 else ("<array of %d>" % n, f.seek(0, 1))[0]
        return [_read_value(f, et) for _ in range(n)]
    raise GgufError("unknown GGUF value type %d" % t)


def dequantize(raw: np.ndarray, ggml_type: int, shape) -> np.ndarray:
    """Raw bytes of one tensor -> float32 array of ``shape`` (row-major, innermost dimension last)."""
    name, bs, bb = GGML[ggml_type]
    n = int(np.prod(shape))
    if name == "F32":
        return raw.view(np.float32)[:n].reshape(shape).copy()
    if name == "F16":
        return raw.view(np.float16)[:n].astype(np.float32).reshape(shape)
    if name == "BF16":
        return (raw.view(np.uint16)[:n].astype(np.uint32) << 16).view(np.float32).reshape(shape)
    blocks = raw[: (n // bs) * bb].reshape(-1, bb)
    d = blocks[:, :2].copy().view(np.float16).astype(np.float32)                     # [nb, 1]
    if name == "Q8_0":
        q = blocks[:, 2:].copy().view(np.int8).astype(np.float32)
        return (q * d).reshape(shape)
    if name == "Q4_0":
        qs = blocks[:, 2:]
        lo, hi = (qs & 0x0F).astype(np.float32) - 8.0, (qs >> 4).astype(np.float32) - 8.0
        return (np.concatenate([lo, hi], 1) * d).reshape(shape)                      # low nibbles are elements 0..15, high 16..31
    if name == "Q4_1":
        m = blocks[:, 2:4].copy().view(np.float16).astype(np.float32)
        qs = blocks[:, 4:]
        lo, hi = (qs & 0x0F).astype(np.float32), (qs >> 4).astype(np.float32)
        return (np.concatenate([lo, hi], 1) * d + m).reshape(shape)
    raise GgufError("tensor type %s is not supported" % name)


def read_gguf(path: str) -> Tuple[Dict[str, Any], Dict[str, np.ndarray]]:
    """-> (metadata, {tensor name: float32 array in [out, in] orientation})."""
    with open(path, "rb") as f:
        if f.read(4) != GGUF_MAGIC:
            raise GgufError("%s is not a GGUF file" % path)
        (version,) = struct.unpack("<I", f.read(4))
        if version < 2:
            raise GgufError("GGUF version %d is not supported" % version)
        n_tensors, n_kv = struct.unpack("<QQ", f.read(16))
        meta: Dict[str, Any] = {}
        for _ in range(n_kv):
            key = _read_str(f)
            (t,) = struct.unpack("<I", f.read(4))
            meta[key] = _read_value(f, t)
        infos = []
        for _ in range(n_tensors):
            name = _read_str(f)
            (nd,) = struct.unpack("<I", f.read(4))
            dims = struct.unpack("<%dQ" % nd, f.read(8 * nd))
            ttype, offset = struct.unpack("<IQ", f.read(12))
            infos.append((name, dims, ttype, offset))
        align = int(meta.get("general.alignment", 32))
        base = (f.tell() + align - 1) // align * align
        tensors = {}
        for name, dims, ttype, offset in infos:
            if ttype not in GGML:
                raise GgufError("tensor %s has unsupported ggml type %d" % (name, ttype))
            _, bs, bb = GGML[ttype]
            n = int(np.prod(dims))
            f.seek(base + offset)
            raw = np.frombuffer(f.read(n // bs * bb), dtype=np.uint8)
            shape = tuple(reversed(dims))          # ggml lists the innermost dimension first
            tensors[name] = dequantize(raw, ttype, shape)
    return meta, tensors


def _unpermute(w: np.ndarray, n_head: int) -> np.ndarray:
    """Inverse of llama.cpp's row permutation of q/k projections (interleaved -> half-rotate rotary layout)."""
    out, inp = w.shape
    return w.reshape(n_head, out // n_head // 2, 2, inp).swapaxes(1, 2).reshape(out, inp)


def convert(path: str, compress: Optional[str] = None, stateful: bool = True):
    """GGUF file -> ``Model`` (stateful decoder). ``compress``: None (float weights) | "int4" | "int8"."""
    import torch
    from ..models.llm_config import LlmConfig
    from ..models.ov_builders import build_llama
    meta, t = read_gguf(path)
    arch = meta.get("general.architecture", "llama")
    if arch not in ("llama", "mistral", "qwen2"):
        raise GgufError("architecture '%s' has no builder" % arch)
    g = lambda k, d=None: meta.get("%s.%s" % (arch, k), d)
    H, L = int(g("embedding_length")), int(g("block_count"))
    Hq = int(g("attention.head_count"))
    Hkv = int(g("attention.head_count_kv", Hq))
    D = int(g("attention.key_length", H // Hq))
    emb = t["token_embd.weight"]
    cfg = LlmConfig(name=str(meta.get("general.name", arch)), vocab_size=emb.shape[0], hidden_size=H, num_layers=L, num_heads=Hq, num_kv_heads=Hkv,
                    head_dim=D, ffn_size=int(g("feed_forward_length")), rope_theta=float(g("rope.freq_base", 10000.0)),
                    rms_eps=float(g("attention.layer_norm_rms_epsilon", 1e-5)), weight_format={"int4": "int4", "int8": "int8"}.get(compress, "bf16"),
                    group_size=128 if H % 128 == 0 else 64)
    tt = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    state = {"embed_tokens": tt(emb), "norm": tt(t["output_norm.weight"]), "lm_head": tt(t.get("output.weight", emb))}
    for l in range(L):
        p, b = "layers.%d." % l, "blk.%d." % l
        state[p + "input_layernorm"] = tt(t[b + "attn_norm.weight"])
        state[p + "post_attention_layernorm"] = tt(t[b + "ffn_norm.weight"])
        state[p + "q_proj"] = tt(_unpermute(t[b + "attn_q.weight"], Hq))
        state[p + "k_proj"] = tt(_unpermute(t[b + "attn_k.weight"], Hkv))
        state[p + "v_proj"] = tt(t[b + "attn_v.weight"])
        state[p + "o_proj"] = tt(t[b + "attn_output.weight"])
        state[p + "gate_proj"] = tt(t[b + "ffn_gate.weight"])
        state[p + "up_proj"] = tt(t[b + "ffn_up.weight"])
        state[p + "down_proj"] = tt(t[b + "ffn_down.weight"])
    model = build_llama(cfg, state, compress=compress, stateful=stateful)
    for k in ("general.name", "general.architecture", "tokenizer.ggml.model", "tokenizer.ggml.bos_token_id", "tokenizer.ggml.eos_token_id"):
        if k in meta and not isinstance(meta[k], list):
            model.set_rt_info(str(meta[k]), ["gguf", k.replace(".", "_")])
    return model
