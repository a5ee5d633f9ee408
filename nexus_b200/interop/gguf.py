"""GGUF v3 writer / reader for llama-family models: metadata key-values, tensor table, 32-byte aligned
data; tensor types F32, F16, Q8_0 and Q4_0 (blocks of 32: FP16 scale + codes).  Q / K projection rows are
permuted between the rotate-half RoPE layout used here (and by HF) and the interleaved-pair layout of
llama.cpp.  Parity: include/nexus/interop/gguf.hpp, src/interop/gguf.cpp of the reference."""
from __future__ import annotations

import struct
from typing import Dict, List, Tuple

import numpy as np
import torch

MAGIC, VERSION, ALIGN = b"GGUF", 3, 32
T_F32, T_F16, T_Q4_0, T_Q8_0 = 0, 1, 2, 8
_VT = {"u8": 0, "i8": 1, "u16": 2, "i16": 3, "u32": 4, "i32": 5, "f32": 6, "bool": 7, "str": 8, "arr": 9, "u64": 10,
       "i64": 11, "f64": 12}
_FMT = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
QK = 32


# ------------------------------------------------------------------------------------------ quantisation
def quantize_q8_0(x: np.ndarray) -> bytes:
    x = np.asarray(x, dtype=np.float32).reshape(-1, QK)
    d = np.abs(x).max(axis=1) / 127.0
    inv = np.where(d > 0, 1.0 / np.where(d > 0, d, 1), 0.0)
    q = np.clip(np.rint(x * inv[:, None]), -127, 127).astype(np.int8)
    out = np.empty((x.shape[0], 2 + QK), dtype=np.uint8)
    out[:, :2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(np.uint8)
    return out.tobytes()


def dequantize_q8_0(raw: bytes, n: int) -> np.ndarray:
    b = np.frombuffer(raw, dtype=np.uint8).reshape(-1, 2 + QK)
    d = b[:, :2].copy().view(np.float16).astype(np.float32)
    return (b[:, 2:].view(np.int8).astype(np.float32) * d).reshape(-1)[:n]


def quantize_q4_0(x: np.ndarray) -> bytes:
    x = np.asarray(x, dtype=np.float32).reshape(-1, QK)
    idx = np.abs(x).argmax(axis=1)
    mx = x[np.arange(x.shape[0]), idx]                 # signed value of largest magnitude
    d = mx / -8.0
    inv = np.where(d != 0, 1.0 / np.where(d != 0, d, 1), 0.0)
    q = np.clip(np.floor(x * inv[:, None] + 8.5), 0, 15).astype(np.uint8)
    out = np.empty((x.shape[0], 2 + QK // 2), dtype=np.uint8)
    out[:, :2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q[:, :16] | (q[:, 16:] << 4)          # low nibble: elements 0..15, high: 16..31
    return out.tobytes()


def dequantize_q4_0(raw: bytes, n: int) -> np.ndarray:
    b = np.frombuffer(raw, dtype=np.uint8).reshape(-1, 2 + QK // 2)
    d = b[:, :2].copy().view(np.float16).astype(np.float32)
    lo, hi = (b[:, 2:] & 15).astype(np.float32) - 8, (b[:, 2:] >> 4).astype(np.float32) - 8
    return (np.concatenate([lo, hi], axis=1) * d).reshape(-1)[:n]


def permute_qk(w: torch.Tensor, heads: int, inverse: bool = False) -> torch.Tensor:
    """Rows of a Q/K projection: rotate-half layout (first half | second half per head) <-> interleaved
    pairs (llama.cpp).  ``inverse`` maps back."""
    out_f, in_f = w.shape
    D = out_f // heads
    if inverse:
        return w.view(heads, D // 2, 2, in_f).transpose(1, 2).reshape(out_f, in_f)
    return w.view(heads, 2, D // 2, in_f).transpose(1, 2).reshape(out_f, in_f)


# ------------------------------------------------------------------------------------------ file format
def _s(b: bytes) -> bytes:
    return struct.pack("<Q", len(b)) + b


def _kv(key: str, val) -> bytes:
    out = _s(key.encode())
    if isinstance(val, bool):
        return out + struct.pack("<I?", _VT["bool"], val)
    if isinstance(val, int):
        return out + (struct.pack("<II", _VT["u32"], val) if 0 <= val < 2 ** 32 else struct.pack("<Iq", _VT["i64"], val))
    if isinstance(val, float):
        return out + struct.pack("<If", _VT["f32"], val)
    if isinstance(val, str):
        return out + struct.pack("<I", _VT["str"]) + _s(val.encode())
    if isinstance(val, (list, tuple)):
        if all(isinstance(v, str) for v in val):
            return out + struct.pack("<IIQ", _VT["arr"], _VT["str"], len(val)) + b"".join(_s(v.encode()) for v in val)
        if all(isinstance(v, int) for v in val):
            return out + struct.pack("<IIQ", _VT["arr"], _VT["i32"], len(val)) + struct.pack(f"<{len(val)}i", *val)
        return out + struct.pack("<IIQ", _VT["arr"], _VT["f32"], len(val)) + struct.pack(f"<{len(val)}f", *val)
    raise TypeError(f"unsupported metadata value for {key}: {type(val)}")


def write_gguf(path: str, metadata: Dict[str, object], tensors: List[Tuple[str, torch.Tensor, int]]) -> None:
    """tensors: (name, 2-D or 1-D tensor, ggml type).  Dimensions are written innermost first."""
    infos, blobs, off = [], [], 0
    for name, t, ty in tensors:
        a = t.detach().float().cpu().numpy()
        if ty in (T_Q8_0, T_Q4_0) and a.shape[-1] % QK:
            raise ValueError(f"{name}: row length {a.shape[-1]} is not a multiple of {QK}")
        raw = {T_F32: lambda: a.astype("<f4").tobytes(), T_F16: lambda: a.astype("<f2").tobytes(),
               T_Q8_0: lambda: quantize_q8_0(a), T_Q4_0: lambda: quantize_q4_0(a)}[ty]()
        infos.append(_s(name.encode()) + struct.pack("<I", a.ndim) + struct.pack(f"<{a.ndim}Q", *reversed(a.shape)) +
                     struct.pack("<IQ", ty, off))
        pad = (-len(raw)) % ALIGN
        blobs.append(raw + b"\0" * pad)
        off += len(raw) + pad
    meta = dict(metadata)
    meta.setdefault("general.alignment", ALIGN)
    head = MAGIC + struct.pack("<IQQ", VERSION, len(tensors), len(meta)) + b"".join(_kv(k, v) for k, v in meta.items()) + \
        b"".join(infos)
    head += b"\0" * ((-len(head)) % ALIGN)
    with open(path, "wb") as f:
        f.write(head)
        for b in blobs:
            f.write(b)


class _Rd:
    def __init__(self, b: bytes):
        self.b, self.p = b, 0

    def take(self, fmt: str):
        v = struct.unpack_from(fmt, self.b, self.p)
        self.p += struct.calcsize(fmt)
        return v if len(v) > 1 else v[0]

    def string(self) -> str:
        n = self.take("<Q")
        if n > len(self.b) - self.p:
            raise ValueError("GGUF: string runs past the end of the file")
        s = self.b[self.p: self.p + n].decode("utf-8")
        self.p += n
        return s

    def value(self, ty: int):
        if ty == _VT["str"]:
            return self.string()
        if ty == _VT["arr"]:
            et, n = self.take("<I"), self.take("<Q")
            return [self.value(et) for _ in range(n)]
        if ty not in _FMT:
            raise ValueError(f"GGUF: unknown value type {ty}")
        return self.take(_FMT[ty])


def read_gguf(path: str):
    """Returns (metadata dict, {name: FP32 tensor}, {name: ggml type})."""
    with open(path, "rb") as f:
        raw = f.read()
    if raw[:4] != MAGIC:
        raise ValueError("not a GGUF file")
    r = _Rd(raw)
    r.p = 4
    version, nt, nkv = r.take("<I"), r.take("<Q"), r.take("<Q")
    if version != VERSION:
        raise ValueError(f"GGUF version {version} (only {VERSION} is supported)")
    meta = {}
    for _ in range(nkv):
        k = r.string()
        meta[k] = r.value(r.take("<I"))
    infos = []
    for _ in range(nt):
        name = r.string()
        nd = r.take("<I")
        dims = [r.take("<Q") for _ in range(nd)]
        ty, off = r.take("<I"), r.take("<Q")
        infos.append((name, tuple(reversed(dims)), ty, off))
    align = int(meta.get("general.alignment", ALIGN))
    base = (r.p + align - 1) // align * align
    tensors, types = {}, {}
    for name, shape, ty, off in infos:
        n = int(np.prod(shape)) if shape else 1
        size = {T_F32: 4 * n, T_F16: 2 * n, T_Q8_0: n // QK * (2 + QK), T_Q4_0: n // QK * (2 + QK // 2)}.get(ty)
        if size is None:
            raise ValueError(f"{name}: unsupported ggml type {ty}")
        blob = raw[base + off: base + off + size]
        if len(blob) != size:
            raise ValueError(f"{name}: data runs past the end of the file")
        a = {T_F32: lambda: np.frombuffer(blob, "<f4").astype(np.float32), T_F16: lambda: np.frombuffer(blob, "<f2").astype(np.float32),
             T_Q8_0: lambda: dequantize_q8_0(blob, n), T_Q4_0: lambda: dequantize_q4_0(blob, n)}[ty]()
        tensors[name] = torch.from_numpy(np.array(a, dtype=np.float32).reshape(shape))
        types[name] = ty
    return meta, tensors, types


# ------------------------------------------------------------------------------------------ llama mapping
def export_llama(model, path: str, weight_type: int = T_F16, name: str = "nexus") -> None:
    """`lm.LanguageModel` (llama family) -> GGUF with llama.cpp tensor names."""
    from .hf import to_hf_state
    cfg = model.config
    hf = to_hf_state(model)
    meta = {"general.architecture": "llama", "general.name": name, "llama.block_count": cfg.n_layer,
            "llama.context_length": cfg.max_position, "llama.embedding_length": cfg.d_model,
            "llama.feed_forward_length": cfg.d_ff, "llama.attention.head_count": cfg.n_head,
            "llama.attention.head_count_kv": cfg.kv_heads(), "llama.rope.dimension_count": cfg.hdim(),
            "llama.rope.freq_base": float(cfg.rope_theta), "llama.attention.layer_norm_rms_epsilon": float(cfg.norm_eps),
            "llama.vocab_size": cfg.vocab_size}
    wt = lambda t: weight_type if t.shape[-1] % QK == 0 or weight_type in (T_F32, T_F16) else T_F16   # noqa: E731
    tensors = [("token_embd.weight", hf["model.embed_tokens.weight"], wt(hf["model.embed_tokens.weight"])),
               ("output_norm.weight", hf["model.norm.weight"], T_F32)]
    if "lm_head.weight" in hf:
        tensors.append(("output.weight", hf["lm_head.weight"], wt(hf["lm_head.weight"])))
    for l in range(cfg.n_layer):
        h, g = f"model.layers.{l}.", f"blk.{l}."
        tensors += [(g + "attn_norm.weight", hf[h + "input_layernorm.weight"], T_F32),
                    (g + "ffn_norm.weight", hf[h + "post_attention_layernorm.weight"], T_F32)]
        q = permute_qk(hf[h + "self_attn.q_proj.weight"], cfg.n_head)
        k = permute_qk(hf[h + "self_attn.k_proj.weight"], cfg.kv_heads())
        for gn, t in (("attn_q", q), ("attn_k", k), ("attn_v", hf[h + "self_attn.v_proj.weight"]),
                      ("attn_output", hf[h + "self_attn.o_proj.weight"]), ("ffn_gate", hf[h + "mlp.gate_proj.weight"]),
                      ("ffn_up", hf[h + "mlp.up_proj.weight"]), ("ffn_down", hf[h + "mlp.down_proj.weight"])):
            tensors.append((g + gn + ".weight", t, wt(t)))
    write_gguf(path, meta, tensors)


def import_llama(path: str):
    from ..lm.config import LmConfig
    from .hf import from_hf_state
    meta, t, _ = read_gguf(path)
    if meta.get("general.architecture") != "llama":
        raise ValueError("only the llama architecture is supported")
    cfg = LmConfig(name="llama", vocab_size=int(meta.get("llama.vocab_size", t["token_embd.weight"].shape[0])),
                   n_layer=int(meta["llama.block_count"]), d_model=int(meta["llama.embedding_length"]),
                   n_head=int(meta["llama.attention.head_count"]),
                   n_kv_head=int(meta.get("llama.attention.head_count_kv", meta["llama.attention.head_count"])),
                   d_ff=int(meta["llama.feed_forward_length"]), max_position=int(meta["llama.context_length"]),
                   norm="rmsnorm", norm_eps=float(meta.get("llama.attention.layer_norm_rms_epsilon", 1e-5)), mlp="swiglu",
                   pos="rope", rope_theta=float(meta.get("llama.rope.freq_base", 10000.0)), bias=False,
                   tie_embeddings="output.weight" not in t)
    hf = {"model.embed_tokens.weight": t["token_embd.weight"], "model.norm.weight": t["output_norm.weight"]}
    if "output.weight" in t:
        hf["lm_head.weight"] = t["output.weight"]
    for l in range(cfg.n_layer):
        h, g = f"model.layers.{l}.", f"blk.{l}."
        hf[h + "input_layernorm.weight"] = t[g + "attn_norm.weight"]
        hf[h + "post_attention_layernorm.weight"] = t[g + "ffn_norm.weight"]
        hf[h + "self_attn.q_proj.weight"] = permute_qk(t[g + "attn_q.weight"], cfg.n_head, inverse=True)
        hf[h + "self_attn.k_proj.weight"] = permute_qk(t[g + "attn_k.weight"], cfg.kv_heads(), inverse=True)
        hf[h + "self_attn.v_proj.weight"] = t[g + "attn_v.weight"]
        hf[h + "self_attn.o_proj.weight"] = t[g + "attn_output.weight"]
        hf[h + "mlp.gate_proj.weight"], hf[h + "mlp.up_proj.weight"] = t[g + "ffn_gate.weight"], t[g + "ffn_up.weight"]
        hf[h + "mlp.down_proj.weight"] = t[g + "ffn_down.weight"]
    return from_hf_state(cfg, hf)
