"""GGUF frontend: a file written in llama.cpp's conventions must give the logits of the model it was made from."""
import struct

import numpy as np
import pytest
import torch

import openvino_b200 as ov
from openvino_b200.frontend import gguf
from openvino_b200.models import llama
from openvino_b200.models.llm_config import TINY_LLAMA

CFG = TINY_LLAMA.with_(vocab_size=96, hidden_size=128, num_heads=4, num_kv_heads=2, head_dim=32, ffn_size=256, num_layers=2, rope_theta=10000.0)


def _s(text):
    b = text.encode()
    return struct.pack("<Q", len(b)) + b


def _permute(w, n_head):          # what llama.cpp's converter does to q/k projections
    out, inp = w.shape
    return w.reshape(n_head, 2, out // n_head // 2, inp).swapaxes(1, 2).reshape(out, inp)


def _q8_0(w):
    blocks = w.reshape(-1, 32)
    d = np.abs(blocks).max(1, keepdims=True) / 127.0
    d[d == 0] = 1.0
    q = np.round(blocks / d).astype(np.int8)
    return np.concatenate([d.astype(np.float16).view(np.uint8), q.view(np.uint8)], 1).tobytes()


def write_gguf(path, cfg, state, wtype):
    kv = [("general.architecture", 8, "llama"), ("general.name", 8, "tiny"), ("llama.block_count", 4, cfg.num_layers),
          ("llama.embedding_length", 4, cfg.hidden_size), ("llama.feed_forward_length", 4, cfg.ffn_size),
          ("llama.attention.head_count", 4, cfg.num_heads), ("llama.attention.head_count_kv", 4, cfg.num_kv_heads),
          ("llama.rope.freq_base", 6, cfg.rope_theta), ("llama.attention.layer_norm_rms_epsilon", 6, cfg.rms_eps),
          ("tokenizer.ggml.tokens", 9, ["a", "b"])]
    names = {"token_embd.weight": state["embed_tokens"], "output_norm.weight": state["norm"], "output.weight": state["lm_head"]}
    for l in range(cfg.num_layers):
        p, b = "layers.%d." % l, "blk.%d." % l
        names[b + "attn_norm.weight"] = state[p + "input_layernorm"]
        names[b + "ffn_norm.weight"] = state[p + "post_attention_layernorm"]
        names[b + "attn_q.weight"] = torch.from_numpy(_permute(state[p + "q_proj"].numpy(), cfg.num_heads))
        names[b + "attn_k.weight"] = torch.from_numpy(_permute(state[p + "k_proj"].numpy(), cfg.num_kv_heads))
        for a, h in (("attn_v", "v_proj"), ("attn_output", "o_proj"), ("ffn_gate", "gate_proj"), ("ffn_up", "up_proj"), ("ffn_down", "down_proj")):
            names[b + a + ".weight"] = state[p + h]
    head = b"GGUF" + struct.pack("<IQQ", 3, len(names), len(kv))
    for k, t, v in kv:
        head += _s(k) + struct.pack("<I", t)
        if t == 8:
            head += _s(v)
        elif t == 4:
            head += struct.pack("<I", v)
        elif t == 6:
            head += struct.pack("<f", v)
        else:
            head += struct.pack("<IQ", 8, len(v)) + b"".join(_s(x) for x in v)
    blobs, infos, off = [], b"", 0
    for name, ten in names.items():
        a = ten.numpy().astype(np.float32)
        if a.ndim == 2 and wtype == "q8_0":
            data, tt = _q8_0(a), 8
        elif a.ndim == 2 and wtype == "f16":
            data, tt = a.astype(np.float16).tobytes(), 1
        else:
            data, tt = a.tobytes(), 0
        infos += _s(name) + struct.pack("<I", a.ndim) + struct.pack("<%dQ" % a.ndim, *reversed(a.shape)) + struct.pack("<IQ", tt, off)
        pad = (-len(data)) % 32
        blobs.append(data + b"\0" * pad)
        off += len(data) + pad
    head += infos
    head += b"\0" * ((-len(head)) % 32)
    with open(path, "wb") as f:
        f.write(head + b"".join(blobs))


@pytest.mark.parametrize("wtype,tol", [("f32", 1e-4), ("f16", 5e-3), ("q8_0", 5e-2)])
def test_gguf_llama_round_trip(tmp_path, wtype, tol):
    state = llama.random_float_state(CFG, seed=1, std=0.1)
    path = str(tmp_path / "tiny.gguf")
    write_gguf(path, CFG, state, wtype)
    meta, tensors = gguf.read_gguf(path)
    assert meta["llama.block_count"] == 2 and meta["general.architecture"] == "llama" and "blk.1.ffn_down.weight" in tensors
    m = ov.Core().read_model(path)
    assert m.get_rt_info(["gguf", "general_architecture"]).value == "llama"
    ids = [3, 17, 5, 60, 9]
    out = ov.compile_model(m, "CPU")({"input_ids": np.array([ids]), "attention_mask": np.ones((1, 5), np.int64),
                                      "position_ids": np.arange(5)[None], "beam_idx": np.zeros(1, np.int32)})[0][0]
    ref = llama.reference_logits(CFG, state, torch.tensor(ids)).numpy()
    assert np.abs(out - ref).max() / np.abs(ref).max() < tol


def test_gguf_errors_and_q4(tmp_path):
    bad = tmp_path / "x.gguf"
    bad.write_bytes(b"NOPE" + b"\0" * 32)
    with pytest.raises(gguf.GgufError):
        gguf.read_gguf(str(bad))
    # Q4_0 block: scale 0.5, nibbles 0..15 twice -> (q - 8) * 0.5
    qs = bytes((i & 15) | ((15 - (i & 15)) << 4) for i in range(16))
    raw = np.frombuffer(np.float16(0.5).tobytes() + qs, dtype=np.uint8)
    vals = gguf.dequantize(raw, 2, (32,))
    np.testing.assert_allclose(vals[:16], (np.arange(16) - 8) * 0.5)
    np.testing.assert_allclose(vals[16:], (15 - np.arange(16) - 8) * 0.5)
