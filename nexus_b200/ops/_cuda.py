"""ctypes bindings of ``lib/libnexus_b200_cuda.so`` (the hand-written sm_100a kernels).

Each wrapper takes torch CUDA tensors, passes raw device pointers plus the current torch stream to
the C entry point and raises on a non-zero return code.  There is no silent fallback: on a machine
with a GPU a missing library is an error.  Bounded waits inside the tensor-core kernels report
through a per-device status word, read with :func:`check_status`.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path
from typing import Dict, Tuple, Optional

import torch

_LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libnexus_b200_cuda.so"
_lib = None
_status = {}
_scratch = {}
launch_count = 0  # kernels launched through this module (bench.py reports it)

BF16, F32, F16, E4M3, E5M2 = 0, 1, 2, 3, 4
ACT = {None: 0, "none": 0, "gelu": 1, "relu": 2, "dgelu": 3, "silu": 4}
_DT = {torch.bfloat16: BF16, torch.float32: F32, torch.float16: F16}
if hasattr(torch, "float8_e4m3fn"):
    _DT[torch.float8_e4m3fn] = E4M3
    _DT[torch.float8_e5m2] = E5M2
_FP8 = tuple(t for t in (getattr(torch, "float8_e4m3fn", None), getattr(torch, "float8_e5m2", None)) if t is not None)


class GemmArgs(C.Structure):
    _fields_ = [
        ("a", C.c_void_p), ("b", C.c_void_p), ("out", C.c_void_p), ("bias", C.c_void_p),
        ("aux_in", C.c_void_p), ("aux_out", C.c_void_p), ("residual", C.c_void_p),
        ("workspace", C.c_void_p), ("status", C.c_void_p),
        ("lda", C.c_int64), ("ldb", C.c_int64), ("ldo", C.c_int64), ("ld_aux", C.c_int64), ("ld_res", C.c_int64),
        ("stride_a", C.c_int64), ("stride_b", C.c_int64), ("stride_o", C.c_int64),
        ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32), ("batch", C.c_int32),
        ("a_mn_major", C.c_int32), ("b_mn_major", C.c_int32),
        ("in_dtype", C.c_int32), ("out_dtype", C.c_int32), ("bias_dtype", C.c_int32), ("res_dtype", C.c_int32),
        ("act", C.c_int32), ("accumulate", C.c_int32), ("split_k", C.c_int32), ("block_n", C.c_int32),
        ("alpha", C.c_float), ("max_ctas", C.c_int32), ("b_dtype_plus1", C.c_int32),
        ("scale_a", C.c_void_p), ("scale_b", C.c_void_p), ("amax_out", C.c_void_p),
    ]


class AttnView(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("row_stride", C.c_int64), ("head_stride", C.c_int64),
                ("batch_stride", C.c_int64)]


class AttnArgs(C.Structure):
    _fields_ = [
        ("q", AttnView), ("k", AttnView), ("v", AttnView), ("o", AttnView),
        ("d_o", AttnView), ("dq", AttnView), ("dk", AttnView), ("dv", AttnView),
        ("lse", C.c_void_p), ("dsum", C.c_void_p), ("status", C.c_void_p),
        ("batch", C.c_int32), ("heads", C.c_int32), ("kv_heads", C.c_int32), ("tq", C.c_int32), ("tk", C.c_int32),
        ("head_dim", C.c_int32), ("causal", C.c_int32), ("window", C.c_int32), ("scale", C.c_float),
        ("merge_o", C.c_void_p), ("merge_lse", C.c_void_p),
        ("softcap", C.c_float), ("alibi_slopes", C.c_void_p),
        ("dropout_p", C.c_float), ("dropout_seed", C.c_uint64), ("dropout_offset", C.c_uint64),
    ]


class OptState(C.Structure):
    _fields_ = [
        ("local_sq", C.c_double), ("lr", C.c_float), ("weight_decay", C.c_float), ("beta1", C.c_float),
        ("beta2", C.c_float), ("eps", C.c_float), ("max_grad_norm", C.c_float), ("loss_scale", C.c_float),
        ("grad_norm", C.c_float), ("clip_coef", C.c_float), ("inv_bias1", C.c_float), ("inv_bias2", C.c_float),
        ("step", C.c_int32), ("found_inf", C.c_int32), ("skipped", C.c_int32), ("good_steps", C.c_int32),
        ("reserved", C.c_int32),
    ]


class AdamChunk(C.Structure):
    _fields_ = [("offset", C.c_int64), ("count", C.c_int64), ("wd_scale", C.c_float), ("lr_scale", C.c_float)]


def available() -> bool:
    return torch.cuda.is_available() and _LIB_PATH.exists()


def lib():
    """Load the kernel library (once).  Raises when it has not been built."""
    global _lib
    if _lib is None:
        path = _LIB_PATH
        if os.environ.get("NEXUS_B200_DEBUG_BOUNDS", "0") == "1":   # kernels with the index checks compiled in
            path = _LIB_PATH.with_name("libnexus_b200_cuda_dbg.so")
        if os.environ.get("NEXUS_B200_CUDA_LIB"):                   # another build of the same library (A/B timing)
            path = Path(os.environ["NEXUS_B200_CUDA_LIB"])
        if not path.exists():
            raise RuntimeError(
                f"{path} is missing: build it with `python -m nexus_b200._build` "
                "(the sm_100a kernels are required on a GPU machine; there is no fallback)")
        _lib = C.CDLL(str(path))
        _lib.nx_gemm_workspace_bytes.restype = C.c_size_t
        _lib.nx_norm_bwd_scratch_bytes.restype = C.c_size_t
        _lib.nx_ce_state_bytes.restype = C.c_size_t
        _lib.nx_colsum_scratch_bytes.restype = C.c_size_t
        _lib.nx_grad_norm_partials.restype = C.c_int64
        _lib.nx_grad_norm_partials.argtypes = [C.c_int64]
    return _lib


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t: Optional[torch.Tensor]) -> C.c_void_p:
    return C.c_void_p(0 if t is None else t.data_ptr())


_KERNELS_PER_CALL = {"nx_norm_bwd": 2, "nx_embedding_bwd": 2, "nx_cross_entropy_shifted": 3, "nx_grad_norm": 2,
                     "nx_colsum": 2, "nx_attention_bwd": 2}


def _check(rc: int, what: str) -> None:
    global launch_count
    launch_count += _KERNELS_PER_CALL.get(what, 1)
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")


def status_word(device=None) -> torch.Tensor:
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    t = _status.get(dev)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=dev)
        _status[dev] = t
    return t


def check_status(device=None) -> None:
    """Synchronises and raises when a bounded wait inside a kernel ran out."""
    code = int(status_word(device).item())
    if code != 0:
        status_word(device).zero_()
        names = {1: "TMA producer", 2: "MMA issuer", 3: "epilogue", 4: "peer", 5: "bad argument",
                 6: "tile index out of range (debug-build bounds check)"}
        raise RuntimeError(f"kernel wait timed out / failed in role: {names.get(code, code)}")


def scratch(nbytes: int, tag: str = "default", device=None) -> torch.Tensor:
    """Grow-only per-(device, tag) scratch buffer (uint8)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = (dev, tag)
    t = _scratch.get(key)
    if t is None or t.numel() < nbytes:
        t = torch.empty(max(int(nbytes), 1 << 20), dtype=torch.uint8, device=dev)
        _scratch[key] = t
    return t


# --------------------------------------------------------------------------------------------- GEMM
_split_cache: Dict[Tuple[int, int, int], int] = {}


def auto_split_k(m: int, n: int, k: int, clusters: int = 74) -> int:
    """Number of K slices that fills the machine best (``split_k=0`` of ``gemm``).

    The pair kernel runs one 256 x 256 tile per cluster of two SMs; a launch of `u` units takes
    ceil(u / clusters) rounds of (k-blocks per unit + a fixed per-unit cost of about six k-blocks for the
    accumulator hand-over and the reduction into the output).  Problems with at least two full rounds of
    tiles are left alone.
    """
    key = (m, n, k)
    s = _split_cache.get(key)
    if s is None:
        if m >= 256 and n >= 256:
            tiles = -(-m // 256) * -(-n // 256)
        else:                     # single-CTA tiles of 128 x (256 | 128) on every SM
            tiles = -(-m // 128) * -(-n // (256 if n >= 256 else 128))
            clusters = 2 * clusters
        kb = -(-k // 64)
        best, s = None, 1
        if tiles < 2 * clusters:
            for cand in range(1, min(16, kb) + 1):
                cost = -(-tiles * cand // clusters) * (-(-kb // cand) + 6)
                if best is None or cost < best:
                    best, s = cost, cand
        _split_cache[key] = s
    return s


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         bias: Optional[torch.Tensor] = None, act: Optional[str] = None,
         aux_in: Optional[torch.Tensor] = None, aux_out: Optional[torch.Tensor] = None,
         residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
         out_dtype: Optional[torch.dtype] = None, accumulate: bool = False, alpha: float = 1.0,
         split_k: int = 1, block_n: int = 0, max_ctas: int = 0, deterministic: bool = False,
         scale_a: Optional[torch.Tensor] = None, scale_b: Optional[torch.Tensor] = None,
         amax_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out = epilogue(alpha * A @ B^T)`` with A logical [M, K], B logical [N, K].

    ``a_mn`` / ``b_mn``: the operand is stored transposed ([K, M] / [K, N], i.e. reduction-major).
    2-D operands, or 3-D for a strided batch.  Rows must be contiguous; row pitch a multiple of 8.
    """
    batched = a.dim() == 3
    if batched:
        batch = a.shape[0]
        ar, ac = a.shape[1], a.shape[2]
        br, bc = b.shape[1], b.shape[2]
    else:
        batch = 1
        ar, ac = a.shape
        br, bc = b.shape
    m, k = (ac, ar) if a_mn else (ar, ac)
    n, kb = (bc, br) if b_mn else (br, bc)
    if k != kb:
        raise ValueError(f"gemm: reduction sizes differ ({k} vs {kb})")
    if a.stride(-1) != 1 or b.stride(-1) != 1:
        raise ValueError("gemm: innermost stride must be 1")
    fp8 = a.dtype in _FP8
    if fp8:
        if b.dtype not in _FP8 or a_mn or b_mn:
            raise ValueError("gemm: 8-bit operands must both be FP8 and K-major")
    elif a.dtype != b.dtype or a.dtype not in (torch.bfloat16, torch.float16):
        raise ValueError("gemm: operands must both be bf16 or fp16 (or both FP8)")
    if out is None:
        od = out_dtype or (torch.bfloat16 if fp8 else a.dtype)
        out = torch.empty((batch, m, n) if batched else (m, n), dtype=od, device=a.device)
    g = GemmArgs()
    g.a, g.b, g.out = a.data_ptr(), b.data_ptr(), out.data_ptr()
    g.lda, g.ldb, g.ldo = a.stride(-2), b.stride(-2), out.stride(-2)
    if batched:
        g.stride_a, g.stride_b, g.stride_o = a.stride(0), b.stride(0), out.stride(0)
    g.m, g.n, g.k, g.batch = m, n, k, batch
    g.a_mn_major, g.b_mn_major = int(a_mn), int(b_mn)
    g.in_dtype, g.out_dtype = _DT[a.dtype], _DT[out.dtype]
    if fp8:
        g.b_dtype_plus1 = _DT[b.dtype] + 1
    if scale_a is not None:
        g.scale_a = scale_a.data_ptr()
    if scale_b is not None:
        g.scale_b = scale_b.data_ptr()
    if amax_out is not None:
        g.amax_out = amax_out.data_ptr()
    if bias is not None:
        g.bias, g.bias_dtype = bias.data_ptr(), _DT[bias.dtype]
    if aux_in is not None:
        g.aux_in, g.ld_aux = aux_in.data_ptr(), aux_in.stride(-2)
    if aux_out is not None:
        g.aux_out, g.ld_aux = aux_out.data_ptr(), aux_out.stride(-2)
    if residual is not None:
        g.residual, g.ld_res, g.res_dtype = residual.data_ptr(), residual.stride(-2), _DT[residual.dtype]
    g.act = ACT[act]
    g.accumulate = int(accumulate)
    g.alpha = alpha
    g.block_n = block_n
    g.max_ctas = max_ctas
    g.status = status_word(a.device).data_ptr()
    L = lib()
    if split_k == 0:
        split_k = auto_split_k(m, n, k) if (not batched and not fp8) else 1
    if split_k > 1 and (aux_in is not None or aux_out is not None or scale_a is not None or scale_b is not None or
                        amax_out is not None or (residual is not None and residual.data_ptr() != out.data_ptr()) or
                        act in ("dgelu",)):
        split_k = 1      # epilogues that only the GEMM itself can apply
    if split_k > 1 and not batched:
        kb_total = (k + 63) // 64
        split_k = min(split_k, kb_total)
        per = (kb_total + split_k - 1) // split_k
        split_k = (kb_total + per - 1) // per
    if split_k > 1 and not batched and accumulate and out.dtype == torch.float32 and not deterministic:
        # slices add into the FP32 output with vector reductions (summation order not fixed)
        g.split_k = split_k
        g.accumulate = 2
        _check(L.nx_gemm(C.byref(g), _stream()), "nx_gemm")
    elif split_k > 1 and not batched:
        # slices go to an FP32 workspace; the reduction pass sums them in a fixed order and applies bias / activation /
        # the add into `out` (a residual that IS `out` counts as accumulate)
        ws = scratch(split_k * m * n * 4, "gemm_splitk", a.device)
        g.workspace = ws.data_ptr()
        g.split_k = split_k
        acc = bool(accumulate) or (residual is not None)
        g.bias, g.residual, g.act, g.accumulate = None, None, ACT["none"], 0
        _check(L.nx_gemm(C.byref(g), _stream()), "nx_gemm")
        _check(L.nx_splitk_reduce_epilogue(C.c_void_p(ws.data_ptr()), _p(out), C.c_int(_DT[out.dtype]),
                                           C.c_int64(out.stride(-2)), C.c_int(m), C.c_int(n), C.c_int(split_k),
                                           C.c_int(int(acc)), _p(bias), C.c_int(_DT[bias.dtype] if bias is not None else F32),
                                           C.c_int(ACT[act]), _stream()), "nx_splitk_reduce")
    else:
        g.split_k = 1
        _check(L.nx_gemm(C.byref(g), _stream()), "nx_gemm")
    return out


# -------------------------------------------------------------------------------------------- norms
def norm_fwd(x, gamma, beta=None, *, rms=False, eps=1e-5, residual=None, sum_out=None, out_dtype=None,
             want_stats=True):
    rows, cols = x.numel() // x.shape[-1], x.shape[-1]
    y = torch.empty(x.shape, dtype=out_dtype or x.dtype, device=x.device)
    mean = torch.empty(rows, dtype=torch.float32, device=x.device) if (want_stats and not rms) else None
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device) if want_stats else None
    _check(lib().nx_norm_fwd(C.c_int(int(rms)), _p(x), C.c_int(_DT[x.dtype]), _p(residual), _p(sum_out), _p(gamma),
                             _p(beta), C.c_int(_DT[gamma.dtype]), _p(y), C.c_int(_DT[y.dtype]), _p(mean), _p(rstd),
                             C.c_int(rows), C.c_int(cols), C.c_float(eps), _stream()), "nx_norm_fwd")
    return y, mean, rstd


def norm_bwd(dy, x, gamma, mean, rstd, *, rms=False, add=None, dx_dtype=None, dgamma=None, dbeta=None,
             accumulate_params=False, want_dx=True, dx=None, dx_lp=None, dx_colsum=None):
    """``dx_colsum`` ([cols] fp32): column sums of the BF16 copy ``dx_lp`` from the same pass - the bias gradient of
    the linear layer that ``dx_lp`` is the output gradient of (accumulated when ``accumulate_params``)."""
    rows, cols = x.numel() // x.shape[-1], x.shape[-1]
    if dx is None and want_dx:
        dx = torch.empty(x.shape, dtype=dx_dtype or x.dtype, device=x.device)
    need_params = dgamma is not None or dbeta is not None or dx_colsum is not None
    L = lib()
    sc = None
    if need_params:
        sc = scratch(L.nx_norm_bwd_scratch_bytes(C.c_int(rows), C.c_int(cols)), "norm_bwd", x.device)
    rc = L.nx_norm_bwd_colsum(C.c_int(int(rms)), _p(dy), C.c_int(_DT[dy.dtype]), _p(x), C.c_int(_DT[x.dtype]), _p(gamma),
                              C.c_int(_DT[gamma.dtype]), _p(mean), _p(rstd), _p(add), _p(dx),
                              C.c_int(_DT[dx.dtype] if dx is not None else F32), _p(dx_lp), _p(dgamma), _p(dbeta),
                              _p(dx_colsum), C.c_int(int(accumulate_params)), _p(sc), C.c_int(rows), C.c_int(cols),
                              _stream())
    if rc == -4:   # no single-pass instance for this shape: the plain kernels, then a column-sum pass over dx_lp
        norm_bwd(dy, x, gamma, mean, rstd, rms=rms, add=add, dgamma=dgamma, dbeta=dbeta,
                 accumulate_params=accumulate_params, dx=dx, dx_lp=dx_lp)
        colsum(dx_lp.view(rows, cols), out=dx_colsum, accumulate=accumulate_params)
        return dx
    _check(rc, "nx_norm_bwd")
    return dx


# ---------------------------------------------------------------------------------------- embedding
def embedding_pos_fwd(tokens, wte, wpe=None, positions=None, out_dtype=torch.float32, seq_len=None):
    rows = tokens.numel()
    cols = wte.shape[1]
    T = seq_len or tokens.shape[-1]
    out = torch.empty(tuple(tokens.shape) + (cols,), dtype=out_dtype, device=wte.device)
    _check(lib().nx_embedding_pos_fwd(_p(tokens), _p(positions), _p(wte), _p(wpe), C.c_int(_DT[wte.dtype]), _p(out),
                                      C.c_int(_DT[out.dtype]), C.c_int64(rows), C.c_int(T), C.c_int(cols),
                                      _stream()), "nx_embedding_pos_fwd")
    return out


def embedding_bwd(tokens, dx, dwte, dwpe, batch, seq_len, deterministic=True):
    cols = dx.shape[-1]
    st = order = None
    if deterministic and dwte is not None:
        flat = tokens.reshape(-1)
        st, order = torch.sort(flat.to(torch.int64), stable=True)
        st = st.to(torch.int32)
    _check(lib().nx_embedding_bwd(_p(tokens), _p(st), _p(order), _p(dx), C.c_int(_DT[dx.dtype]), _p(dwte), _p(dwpe),
                                  C.c_int(batch), C.c_int(seq_len), C.c_int(cols), _stream()), "nx_embedding_bwd")


# ------------------------------------------------------------------------------------ cross-entropy
def cross_entropy_shifted(logits, tokens, *, targets=None, vocab=None, ignore_index=-100, smoothing=0.0,
                          z_loss=0.0, grad_scale=1.0, write_grad=True, loss_out=None, loss_weight=1.0,
                          accumulate_loss=False, seq_len=None, grad_scale_dev=None):
    """In-place fused CE.  ``logits`` [rows, ld] becomes d(loss*grad_scale)/dlogits.  Returns the loss
    tensor (1 element, device).  ``grad_scale_dev``: a 1-element FP32 device tensor that multiplies the gradient too
    (the dynamic loss scale inside the optimizer state)."""
    L = lib()
    rows, ld = logits.shape[0], logits.stride(0)
    vocab = vocab or logits.shape[1]
    T = seq_len or tokens.shape[-1]
    row_loss = scratch(rows * 4, "ce_rows", logits.device)
    state = scratch(int(L.nx_ce_state_bytes()), "ce_state", logits.device)
    if loss_out is None:
        loss_out = torch.empty(1, dtype=torch.float32, device=logits.device)
    _check(L.nx_cross_entropy_shifted_scaled(_p(logits), C.c_int(_DT[logits.dtype]), _p(tokens), _p(targets),
                                             _p(row_loss), _p(state), _p(loss_out), C.c_float(loss_weight),
                                             C.c_int(int(accumulate_loss)), C.c_int64(rows), C.c_int(T), C.c_int(vocab),
                                             C.c_int64(ld), C.c_int(ignore_index), C.c_float(smoothing),
                                             C.c_float(z_loss), C.c_float(grad_scale), _p(grad_scale_dev),
                                             C.c_int(int(write_grad)), _stream()),
           "nx_cross_entropy_shifted")
    return loss_out


# ------------------------------------------------------------------------------------------ dropout
def dropout(x, p, seed, offset, out=None):
    out = torch.empty_like(x) if out is None else out
    _check(lib().nx_dropout(_p(x), _p(out), C.c_int(_DT[x.dtype]), C.c_int64(x.numel()), C.c_float(p),
                            C.c_uint64(seed), C.c_uint64(offset), C.c_int(0), _stream()), "nx_dropout")
    return out


def philox_uniform(n, seed, offset, device="cuda"):
    out = torch.empty(n, dtype=torch.float32, device=device)
    _check(lib().nx_philox_uniform(_p(out), C.c_int64(n), C.c_uint64(seed), C.c_uint64(offset), _stream()),
           "nx_philox_uniform")
    return out


# ---------------------------------------------------------------------------------------- optimizer
def opt_state_tensor(device="cuda") -> torch.Tensor:
    return torch.zeros(C.sizeof(OptState), dtype=torch.uint8, device=device)


def pack_opt_state(**kw) -> bytes:
    s = OptState()
    for k, v in kw.items():
        setattr(s, k, v)
    return bytes(s)


def unpack_opt_state(raw: bytes) -> OptState:
    return OptState.from_buffer_copy(raw)


def make_chunks(segments, chunk=1 << 16, device="cuda") -> torch.Tensor:
    """segments: iterable of (offset, count, wd_scale, lr_scale) -> device chunk table (uint8 tensor)."""
    items = []
    for off, cnt, wd, lr in segments:
        pos = 0
        while pos < cnt:
            c = min(chunk, cnt - pos)
            items.append(AdamChunk(off + pos, c, wd, lr))
            pos += c
    arr = (AdamChunk * len(items))(*items)
    t = torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8).to(device)
    t.nchunks = len(items)
    return t


def grad_norm(grad, state, *, extra_sq=None, local_only=False):
    L = lib()
    n = grad.numel()
    parts = scratch(int(L.nx_grad_norm_partials(n)) * 8, "gnorm", grad.device)
    _check(L.nx_grad_norm(_p(grad), C.c_int(_DT[grad.dtype]), C.c_int64(n), _p(parts), _p(state), _p(extra_sq),
                          C.c_int(int(local_only)), _stream()), "nx_grad_norm")


def adamw(master, grad, m, v, shadow, chunks, state, *, zero_grad=False, sr_seed=0, nchunks=None):
    _check(lib().nx_adamw(_p(master), _p(grad), C.c_int(_DT[grad.dtype]), _p(m), _p(v), _p(shadow),
                          C.c_int(_DT[shadow.dtype] if shadow is not None else BF16), _p(chunks),
                          C.c_int(nchunks if nchunks is not None else chunks.nchunks), _p(state),
                          C.c_int(int(zero_grad)), C.c_uint64(sr_seed), _stream()), "nx_adamw")


def loss_scale_update(state, growth=2.0, backoff=0.5, interval=2000, min_scale=1.0, max_scale=65536.0 ** 2):
    _check(lib().nx_loss_scale_update(_p(state), C.c_float(growth), C.c_float(backoff), C.c_int(interval),
                                      C.c_float(min_scale), C.c_float(max_scale), _stream()),
           "nx_loss_scale_update")


def count_nonfinite(x) -> torch.Tensor:
    cnt = torch.zeros(1, dtype=torch.int32, device=x.device)
    _check(lib().nx_count_nonfinite(_p(x), C.c_int(_DT[x.dtype]), C.c_int64(x.numel()), _p(cnt), _stream()),
           "nx_count_nonfinite")
    return cnt


def colsum(dy, out=None, accumulate=False):
    rows, cols = dy.shape
    L = lib()
    if out is None:
        out = torch.empty(cols, dtype=torch.float32, device=dy.device)
    sc = scratch(int(L.nx_colsum_scratch_bytes(C.c_int(rows), C.c_int(cols))), "colsum", dy.device)
    _check(L.nx_colsum(_p(dy), C.c_int(_DT[dy.dtype]), _p(out), _p(sc), C.c_int(rows), C.c_int(cols),
                       C.c_int64(dy.stride(0)), C.c_int(int(accumulate)), _stream()), "nx_colsum")
    return out


# ---------------------------------------------------------------------------------------- attention
def _view(t: torch.Tensor) -> AttnView:
    # t: [B, T, H, D] (any strides with unit innermost stride)
    if t.stride(3) != 1:
        raise ValueError("attention: innermost stride must be 1")
    return AttnView(t.data_ptr(), t.stride(1), t.stride(2), t.stride(0))


def _alibi_ptr(alibi_slopes, heads, device):
    if alibi_slopes is None:
        return None
    if alibi_slopes.dtype != torch.float32 or alibi_slopes.numel() != heads or not alibi_slopes.is_contiguous() \
            or alibi_slopes.device != device:
        raise ValueError("attention: alibi_slopes must be a contiguous FP32 tensor of [heads] on the same device")
    return alibi_slopes.data_ptr()


def attention_fwd(q, k, v, *, causal=True, window=0, scale=None, out=None, merge_o=None, merge_lse=None,
                  softcap=0.0, alibi_slopes=None, dropout_p=0.0, dropout_seed=0, dropout_offset=0, lse=None):
    """q [B,Tq,H,D], k/v [B,Tk,Hkv,D] bf16 (strided views allowed).  Returns (o, lse[B,H,Tq]).
    ``merge_o`` (FP32 [B,Tq,H,D]) / ``merge_lse`` (FP32 [B,H,Tq]): running result of earlier key/value
    chunks; this chunk is merged into them in the kernel's epilogue (ring / chunked attention)."""
    B, Tq, H, D = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    o = torch.empty((B, Tq, H, D), dtype=q.dtype, device=q.device) if out is None else out
    if lse is None:
        lse = torch.empty((B, H, Tq), dtype=torch.float32, device=q.device)
    a = AttnArgs()
    a.q, a.k, a.v, a.o = _view(q), _view(k), _view(v), _view(o)
    a.lse = lse.data_ptr()
    a.status = status_word(q.device).data_ptr()
    a.batch, a.heads, a.kv_heads, a.tq, a.tk, a.head_dim = B, H, Hkv, Tq, Tk, D
    a.causal, a.window = int(causal), int(window)
    a.scale = scale if scale is not None else D ** -0.5
    a.softcap, a.alibi_slopes = float(softcap), _alibi_ptr(alibi_slopes, H, q.device)
    a.dropout_p, a.dropout_seed, a.dropout_offset = float(dropout_p), int(dropout_seed), int(dropout_offset)
    if merge_o is not None:
        if not (merge_o.is_contiguous() and merge_lse.is_contiguous() and merge_o.dtype == torch.float32):
            raise ValueError("attention_fwd: merge buffers must be contiguous FP32")
        a.merge_o, a.merge_lse = merge_o.data_ptr(), merge_lse.data_ptr()
    _check(lib().nx_attention_fwd(C.byref(a), _stream()), "nx_attention_fwd")
    return o, lse


def attention_bwd(q, k, v, o, lse, d_o, *, causal=True, window=0, scale=None, dq=None, dk=None, dv=None,
                  softcap=0.0, alibi_slopes=None, dropout_p=0.0, dropout_seed=0, dropout_offset=0):
    B, Tq, H, D = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    dq = torch.empty((B, Tq, H, D), dtype=q.dtype, device=q.device) if dq is None else dq
    dk = torch.empty((B, Tk, Hkv, D), dtype=q.dtype, device=q.device) if dk is None else dk
    dv = torch.empty((B, Tk, Hkv, D), dtype=q.dtype, device=q.device) if dv is None else dv
    dsum = torch.empty((B, H, Tq), dtype=torch.float32, device=q.device)
    a = AttnArgs()
    a.q, a.k, a.v, a.o = _view(q), _view(k), _view(v), _view(o)
    a.d_o, a.dq, a.dk, a.dv = _view(d_o), _view(dq), _view(dk), _view(dv)
    a.lse, a.dsum = lse.data_ptr(), dsum.data_ptr()
    a.status = status_word(q.device).data_ptr()
    a.batch, a.heads, a.kv_heads, a.tq, a.tk, a.head_dim = B, H, Hkv, Tq, Tk, D
    a.causal, a.window = int(causal), int(window)
    a.scale = scale if scale is not None else D ** -0.5
    a.softcap, a.alibi_slopes = float(softcap), _alibi_ptr(alibi_slopes, H, q.device)
    a.dropout_p, a.dropout_seed, a.dropout_offset = float(dropout_p), int(dropout_seed), int(dropout_offset)
    _check(lib().nx_attention_bwd(C.byref(a), _stream()), "nx_attention_bwd")
    return dq, dk, dv
