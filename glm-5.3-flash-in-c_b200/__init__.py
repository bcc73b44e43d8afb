"""ctypes binding of libglm53f_b200.so, the sm_100a decode engine for the GLM-5.3-Flash
architecture (C ABI: include/glm53f_b200.h).

This package holds no arithmetic. Every call goes to the CUDA library; if the library has not
been built the import of `lib()` raises, because there is no CPU implementation to fall back
to. The directory name is not a Python identifier, so load it with importlib (see
`__graft_entry__.load_package`), which registers it as ``glm53f_b200``.

Mirrors the host-side surface of josesilva05/glm-5.3-flash-in-c for the decode path:
`Engine` plays the part of `Glm53fModel` + `Glm53fGpu` (src/model/glm53f_model.h:53-75,
src/gpu/glm53f_gpu.h:38-53) and the `op_*` methods the op functions of
include/glm53f/glm53f.h:136-360.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libglm53f_b200.so")

DT_F32, DT_BF16, DT_FP8 = 0, 1, 2


class Config(C.Structure):
    """g5b_config (include/glm53f_b200.h); the reference's Glm53fCfg, glm53f.h:48-95."""
    _fields_ = [
        ("hidden", C.c_int32), ("n_layers", C.c_int32), ("vocab", C.c_int32), ("rms_eps", C.c_float),
        ("hc_mult", C.c_int32), ("hc_iters", C.c_int32), ("hc_eps", C.c_float),
        ("kda_heads", C.c_int32), ("kda_head_dim", C.c_int32), ("conv_k", C.c_int32), ("gate_lb", C.c_float),
        ("mla_heads", C.c_int32), ("q_lora", C.c_int32), ("kv_lora", C.c_int32), ("qk_nope", C.c_int32),
        ("v_head", C.c_int32),
        ("index_topk", C.c_int32), ("index_kpool", C.c_int32), ("index_heads", C.c_int32), ("index_dim", C.c_int32),
        ("n_experts", C.c_int32), ("topk", C.c_int32), ("n_shared", C.c_int32), ("moe_inter", C.c_int32),
        ("dense_inter", C.c_int32), ("routed_scale", C.c_float), ("norm_topk", C.c_int32),
        ("swiglu_limit", C.c_float), ("fp8_block_r", C.c_int32), ("fp8_block_c", C.c_int32),
    ]

    def copy(self) -> "Config":
        c = Config()
        C.memmove(C.byref(c), C.byref(self), C.sizeof(Config))
        return c


class Tensor(C.Structure):
    """g5b_tensor (include/glm53f_b200.h)."""
    _fields_ = [("data", C.c_void_p), ("scale_inv", C.c_void_p), ("dtype", C.c_int32),
                ("rows", C.c_int32), ("cols", C.c_int32), ("on_device", C.c_int32)]


def full_size_config() -> Config:
    """The released checkpoint's text_config (reference config.json; glm53f.h:48-88)."""
    return Config(hidden=4096, n_layers=45, vocab=154880, rms_eps=1e-5, hc_mult=4, hc_iters=20, hc_eps=1e-6,
                  kda_heads=64, kda_head_dim=128, conv_k=4, gate_lb=-5.0, mla_heads=64, q_lora=1536,
                  kv_lora=512, qk_nope=256, v_head=256, index_topk=2048, index_kpool=4, index_heads=32,
                  index_dim=128, n_experts=288, topk=8, n_shared=1, moe_inter=2048, dense_inter=12288,
                  routed_scale=2.5, norm_topk=1, swiglu_limit=10.0, fp8_block_r=128, fp8_block_c=128)


def as_tensor(arr: np.ndarray, dtype: int, scale: np.ndarray | None = None):
    """Wrap a numpy array (float32 / uint16 bf16 bits / uint8 e4m3 codes) as a g5b_tensor.
    Returns (Tensor, keepalive)."""
    a = np.ascontiguousarray(arr)
    want = {DT_F32: np.float32, DT_BF16: np.uint16, DT_FP8: np.uint8}[dtype]
    if a.dtype != want:
        raise TypeError(f"dtype {dtype} needs {want}, got {a.dtype}")
    rows = a.shape[0] if a.ndim >= 1 else 1
    cols = int(a.size // rows) if rows else 0
    s = None
    if dtype == DT_FP8:
        if scale is None:
            raise ValueError("an FP8 tensor needs its scale grid")
        s = np.ascontiguousarray(scale, dtype=np.float32)
    t = Tensor(a.ctypes.data, s.ctypes.data if s is not None else None, dtype, rows, cols, 0)
    return t, (a, s)


_lib = None


def lib() -> C.CDLL:
    """Load libglm53f_b200.so. Raises if it has not been built: there is no fallback."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(f"{LIB_PATH} is missing: build it with __graft_entry__.build(); "
                           "this package has no CPU implementation")
    L = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
    _declare(L, "g5b", C.c_void_p)
    L.g5b_last_error.restype = C.c_char_p
    L.g5b_engine_create.restype = C.c_void_p
    L.g5b_engine_create.argtypes = [C.POINTER(Config), C.c_char_p, C.c_char_p, C.c_int, C.c_int, C.c_int, C.c_int]
    L.g5b_engine_fill_expert.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_uint64, C.c_void_p, C.c_void_p, C.c_void_p]
    L.g5b_engine_fill_matrix.argtypes = [C.c_void_p, C.c_char_p, C.c_int, C.c_uint64, C.c_float, C.c_void_p]
    L.g5b_engine_load_checkpoint.argtypes = [C.c_void_p, C.c_char_p, C.c_int]
    L.g5b_engine_synth_session.argtypes = [C.c_void_p, C.c_uint64, C.c_int]
    L.g5b_engine_last_picks.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
    L.g5b_engine_decode_greedy.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
    L.g5b_engine_ep_handle_bytes.restype = C.c_size_t
    L.g5b_engine_ep_export.argtypes = [C.c_void_p, C.c_void_p]
    L.g5b_engine_ep_connect.argtypes = [C.c_void_p, C.c_void_p]
    L.g5b_engine_ep_resync.argtypes = [C.c_void_p]
    L.g5b_engine_ep_connect_local.argtypes = [C.c_void_p, C.c_int]
    L.g5b_engine_use_sequence.argtypes = [C.c_void_p, C.c_int]
    L.g5b_engine_decode_batch.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    L.g5b_engine_set_option.argtypes = [C.c_void_p, C.c_char_p, C.c_int]
    for fn in ("g5b_dev_moe", "g5b_dev_kda"):
        getattr(L, fn).argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p]
    L.g5b_dev_mla.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
    L.g5b_dev_decoder_layer.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int]
    L.g5b_engine_sync.argtypes = [C.c_void_p]
    L.g5b_engine_stream.restype = C.c_void_p
    L.g5b_engine_stream.argtypes = [C.c_void_p]
    L.g5b_launch_count.restype = C.c_uint64
    L.g5b_rmsnorm_noalloc.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_void_p]
    L.g5b_time_op.argtypes = [C.c_void_p, C.c_char_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_void_p,
                              C.c_int, C.c_size_t, C.c_void_p, C.c_void_p]
    L.g5b_engine_decode_sampled.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_float, C.c_uint64, C.c_void_p]
    L.g5b_sample_host.argtypes = [C.c_void_p, C.c_int, C.c_float, C.c_float, C.c_uint64, C.c_uint64, C.c_void_p, C.c_int]
    L.g5b_time_matvec.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_size_t, C.c_void_p]
    _lib = L
    return L


def _declare(L, prefix: str, handle):
    """argtypes shared by the engine (g5b_), the oracle (orc_) and the reference shim (ref_)."""
    f32p = C.c_void_p
    model = "engine" if prefix == "g5b" else "model"

    def sig(name, args, res=C.c_int):
        fn = getattr(L, f"{prefix}_{name}", None)
        if fn is not None:
            fn.argtypes, fn.restype = args, res

    sig(f"{model}_load", [handle, C.c_char_p, C.POINTER(Tensor)])
    sig(f"{model}_finalize", [handle])
    sig(f"{model}_forward", [handle, C.c_void_p, C.c_int, f32p, C.c_void_p])
    sig(f"{model}_reset", [handle], None)
    sig(f"{model}_free", [handle], None)
    sig(f"{model}_cached", [handle])
    dev = [C.c_int] if prefix == "g5b" else []
    sig("matvec_host", [C.POINTER(Tensor), C.c_int, C.c_int, f32p, C.c_int, f32p] + dev)
    sig("rmsnorm_host", [f32p, f32p, f32p, C.c_int, C.c_int, C.c_float] + dev)
    sig("swiglu_host", [f32p, f32p, C.c_int, C.c_int, C.c_float] + dev)
    sig("shortconv_host", [f32p, f32p, f32p, f32p, C.c_int, C.c_int, C.c_int] + dev)
    sig("op_matvec", [handle, C.c_char_p, f32p, C.c_int, f32p])
    sig("op_hc_pre", [handle, C.c_int, C.c_int, f32p, C.c_int, f32p, f32p, f32p])
    sig("op_hc_post", [handle, f32p, f32p, f32p, f32p, C.c_int])
    sig("op_kda", [handle, C.c_int, f32p, C.c_int, f32p])
    sig("op_mla", [handle, C.c_int, f32p, C.c_int, C.c_int, f32p, C.c_void_p, C.c_void_p])
    sig("op_router", [handle, C.c_int, f32p, C.c_int, C.c_void_p, f32p])
    sig("op_moe", [handle, C.c_int, f32p, C.c_int, f32p, C.c_int])
    sig("op_mlp", [handle, C.c_int, f32p, C.c_int, f32p])
    sig("op_decoder_layer", [handle, C.c_int, f32p, C.c_int, C.c_int])
    sig("state_write", [handle, C.c_int, C.c_int, C.c_size_t, f32p, C.c_size_t])
    sig("state_read", [handle, C.c_int, C.c_int, C.c_size_t, f32p, C.c_size_t])
    sig(f"{model}_enable_mtp", [handle])
    sig("mtp_feed", [handle, f32p, C.c_void_p, C.c_int, C.c_void_p, f32p])
    sig("mtp_hidden", [handle, C.c_int, C.c_int, f32p])


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


class FlatModel:
    """A loaded model behind one of the three flat C APIs (engine, oracle, reference shim).
    Subclasses supply `L` (the CDLL), `prefix`, `handle` and `cfg`."""
    L = None
    prefix = ""
    model_word = "model"

    def _fn(self, name):
        return getattr(self.L, f"{self.prefix}_{name}")

    def _err(self, what):
        msg = ""
        if self.prefix == "g5b":
            msg = (self.L.g5b_last_error() or b"").decode()
        raise RuntimeError(f"{self.prefix}_{what} failed: {msg}")

    # ---- loading
    def load(self, name: str, arr: np.ndarray, dtype: int, scale=None):
        t, keep = as_tensor(arr, dtype, scale)
        if self._fn(f"{self.model_word}_load")(self.handle, name.encode(), C.byref(t)) != 0:
            self._err(f"load({name})")

    def load_all(self, tensors: dict):
        """tensors: name -> (array, dtype, scale-or-None), names below 'model.language_model.'"""
        for name, (arr, dt, sc) in tensors.items():
            self.load(name, arr, dt, sc)

    def finalize(self):
        if self._fn(f"{self.model_word}_finalize")(self.handle) != 0:
            self._err("finalize")

    # ---- model level (glm53f_model_forward, glm53f_model.h:59-64)
    def forward(self, ids, want_logits=True, want_argmax=False):
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        T = int(ids.size)
        logits = np.zeros(self.cfg.vocab, np.float32) if want_logits else None
        am = np.zeros(T, np.int32) if want_argmax else None
        rc = self._fn(f"{self.model_word}_forward")(
            self.handle, ids.ctypes.data, T,
            logits.ctypes.data if logits is not None else None,
            am.ctypes.data if am is not None else None)
        if rc != 0:
            self._err("forward")
        return logits, am

    def reset(self):
        self._fn(f"{self.model_word}_reset")(self.handle)

    # ---- the multi-token-prediction layer (src/model/glm53f_mtp.h)
    def enable_mtp(self):
        """Before loading: the model then also takes the tensors of checkpoint layer n_layers."""
        if self._fn(f"{self.model_word}_enable_mtp")(self.handle) != 0:
            self._err("enable_mtp")

    def mtp_feed(self, next_ids, h=None, want_draft=True):
        """glm53f_mtp_feed: T positions' hidden states (None: the ones the last forward call kept)
        and the tokens that follow them. Returns (draft token or None, the layer's output rows [T][hidden])."""
        ids = np.ascontiguousarray(next_ids, dtype=np.int32)
        T = int(ids.size)
        hp = None
        if h is not None:
            h = _f32(h).reshape(T, self.cfg.hidden)
            hp = h.ctypes.data
        x = np.zeros((T, self.cfg.hidden), np.float32)
        draft = C.c_int(-1)
        if self._fn("mtp_feed")(self.handle, hp, ids.ctypes.data, T, C.addressof(draft) if want_draft else None,
                                x.ctypes.data) != 0:
            self._err("mtp_feed")
        return (int(draft.value) if want_draft else None), x

    def mtp_hidden(self, first: int, T: int) -> np.ndarray:
        out = np.zeros((T, self.cfg.hidden), np.float32)
        if self._fn("mtp_hidden")(self.handle, first, T, out.ctypes.data) != 0:
            self._err("mtp_hidden")
        return out

    @property
    def cached(self) -> int:
        return int(self._fn(f"{self.model_word}_cached")(self.handle))

    # ---- layer ops (glm53f.h:136-360)
    def op_matvec(self, name, x):
        x = _f32(x)
        T = x.shape[0] if x.ndim == 2 else 1
        rows = self._rows_of(name)
        y = np.zeros((T, rows), np.float32)
        if self._fn("op_matvec")(self.handle, name.encode(), x.ctypes.data, T, y.ctypes.data) != 0:
            self._err("op_matvec")
        return y if x.ndim == 2 else y[0]

    def _rows_of(self, name):
        return self._rows[name]

    def op_hc_pre(self, layer, site, h):
        h = _f32(h)
        T, M, E = h.shape
        x = np.zeros((T, E), np.float32); post = np.zeros((T, M), np.float32); comb = np.zeros((T, M * M), np.float32)
        if self._fn("op_hc_pre")(self.handle, layer, site, h.ctypes.data, T, x.ctypes.data,
                                 post.ctypes.data, comb.ctypes.data) != 0:
            self._err("op_hc_pre")
        return x, post, comb

    def op_hc_post(self, h, y, post, comb):
        h = _f32(h).copy(); y = _f32(y); post = _f32(post); comb = _f32(comb)
        if self._fn("op_hc_post")(self.handle, h.ctypes.data, y.ctypes.data, post.ctypes.data,
                                  comb.ctypes.data, h.shape[0]) != 0:
            self._err("op_hc_post")
        return h

    def op_kda(self, layer, x):
        x = _f32(x); out = np.zeros_like(x)
        if self._fn("op_kda")(self.handle, layer, x.ctypes.data, x.shape[0], out.ctypes.data) != 0:
            self._err("op_kda")
        return out

    def op_mla(self, layer, x, cached):
        x = _f32(x); out = np.zeros_like(x)
        sel = np.zeros(self.cfg.index_topk + self.cfg.index_kpool, np.int32)
        n = C.c_int(0)
        if self._fn("op_mla")(self.handle, layer, x.ctypes.data, x.shape[0], cached, out.ctypes.data,
                              sel.ctypes.data, C.addressof(n)) != 0:
            self._err("op_mla")
        return out, (None if n.value < 0 else sel[:n.value].copy())

    def op_router(self, layer, x):
        x = _f32(x); T = x.shape[0]; K = self.cfg.topk
        idx = np.zeros((T, K), np.int32); w = np.zeros((T, K), np.float32)
        if self._fn("op_router")(self.handle, layer, x.ctypes.data, T, idx.ctypes.data, w.ctypes.data) != 0:
            self._err("op_router")
        return idx, w

    def op_moe(self, layer, x, with_shared=True):
        x = _f32(x); out = np.zeros_like(x)
        if self._fn("op_moe")(self.handle, layer, x.ctypes.data, x.shape[0], out.ctypes.data,
                              1 if with_shared else 0) != 0:
            self._err("op_moe")
        return out

    def op_mlp(self, layer, x):
        x = _f32(x); out = np.zeros_like(x)
        if self._fn("op_mlp")(self.handle, layer, x.ctypes.data, x.shape[0], out.ctypes.data) != 0:
            self._err("op_mlp")
        return out

    def op_decoder_layer(self, layer, h, cached):
        h = _f32(h).copy()
        if self._fn("op_decoder_layer")(self.handle, layer, h.ctypes.data, h.shape[0], cached) != 0:
            self._err("op_decoder_layer")
        return h

    def state_write(self, layer, kind, offset, src):
        src = _f32(src)
        if self._fn("state_write")(self.handle, layer, kind, offset, src.ctypes.data, src.size) != 0:
            self._err("state_write")

    def state_read(self, layer, kind, offset, count):
        dst = np.zeros(count, np.float32)
        if self._fn("state_read")(self.handle, layer, kind, offset, dst.ctypes.data, count) != 0:
            self._err("state_read")
        return dst


class Engine(FlatModel):
    """The CUDA engine on one GPU (g5b_engine_*)."""
    prefix = "g5b"
    model_word = "engine"

    def __init__(self, cfg: Config, is_mla, is_dense, cap: int, device: int = 0, ep_rank: int = 0,
                 ep_size: int = 1):
        self.L = lib()
        self.cfg = cfg.copy()
        self.is_mla = bytes(bytearray(int(v) for v in is_mla))
        self.is_dense = bytes(bytearray(int(v) for v in is_dense))
        self.handle = self.L.g5b_engine_create(C.byref(self.cfg), self.is_mla, self.is_dense, cap, device,
                                               ep_rank, ep_size)
        if not self.handle:
            self._err("engine_create")
        self._rows = {}

    def load(self, name, arr, dtype, scale=None):
        super().load(name, arr, dtype, scale)
        self._rows[name] = arr.shape[0]

    def set_option(self, name: str, value: int):
        if self.L.g5b_engine_set_option(self.handle, name.encode(), value) != 0:
            self._err(f"set_option({name})")

    def fill_expert(self, layer, expert, seed, gate_s, up_s, down_s):
        g, u, d = _f32(gate_s), _f32(up_s), _f32(down_s)
        if self.L.g5b_engine_fill_expert(self.handle, layer, expert, seed, g.ctypes.data, u.ctypes.data,
                                         d.ctypes.data) != 0:
            self._err("fill_expert")

    def fill_matrix(self, name: str, dtype: int, seed: int, rows: int, mul: float = 0.0, scale_inv=None):
        """A named matrix generated on the GPU (g5b_engine_fill_matrix); `rows` is recorded for op_matvec."""
        sc = _f32(scale_inv) if scale_inv is not None else None
        if self.L.g5b_engine_fill_matrix(self.handle, name.encode(), dtype, seed, C.c_float(mul),
                                         sc.ctypes.data if sc is not None else None) != 0:
            self._err(f"fill_matrix({name})")
        self._rows[name] = rows

    def load_checkpoint(self, directory: str, threads: int = 4):
        """Stream every tensor this engine owns from a safetensors directory into HBM (C loader)."""
        if self.L.g5b_engine_load_checkpoint(self.handle, directory.encode(), threads) != 0:
            self._err("load_checkpoint")

    def synth_session(self, seed: int, positions: int):
        """Synthetic session state for every sequence at `positions` positions (g5b_engine_synth_session)."""
        if self.L.g5b_engine_synth_session(self.handle, seed, positions) != 0:
            self._err("synth_session")

    def last_picks(self, T: int = 1):
        """(idx [T][topk], w [T][topk]) of the most recent MoE pass (g5b_engine_last_picks)."""
        idx = np.zeros((T, self.cfg.topk), np.int32); w = np.zeros((T, self.cfg.topk), np.float32)
        if self.L.g5b_engine_last_picks(self.handle, T, idx.ctypes.data, w.ctypes.data) != 0:
            self._err("last_picks")
        return idx, w

    def use_sequence(self, seq: int):
        if self.L.g5b_engine_use_sequence(self.handle, seq) != 0:
            self._err("use_sequence")

    def decode_batch(self, ids, want_logits=True):
        """One new token per sequence (option "sequences"): returns (logits [S][vocab] or None, argmax [S])."""
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        S = ids.size
        lg = np.zeros((S, self.cfg.vocab), np.float32) if want_logits else None
        am = np.zeros(S, np.int32)
        if self.L.g5b_engine_decode_batch(self.handle, ids.ctypes.data, lg.ctypes.data if want_logits else None,
                                          am.ctypes.data) != 0:
            self._err("decode_batch")
        return lg, am

    def ep_export(self) -> bytes:
        """This rank's exchange-region handle (g5b_engine_ep_export), to be gathered from all ranks."""
        buf = C.create_string_buffer(self.L.g5b_engine_ep_handle_bytes())
        if self.L.g5b_engine_ep_export(self.handle, buf) != 0:
            self._err("ep_export")
        return buf.raw

    def ep_connect(self, handles):
        """Map every rank's exchange region (handles in rank order, this rank's own included)."""
        blob = b"".join(handles)
        if self.L.g5b_engine_ep_connect(self.handle, blob) != 0:
            self._err("ep_connect")

    @staticmethod
    def ep_connect_local(engines):
        """Wire engines that live in this process, one per device, engines[r] = rank r."""
        arr = (C.c_void_p * len(engines))(*[e.handle for e in engines])
        if engines[0].L.g5b_engine_ep_connect_local(arr, len(engines)) != 0:
            engines[0]._err("ep_connect_local")

    def ep_resync(self):
        """Re-align the ranks' step count after a failed step (collective; barriers are the caller's)."""
        if self.L.g5b_engine_ep_resync(self.handle) != 0:
            self._err("ep_resync")

    def decode_greedy(self, first: int, n: int):
        out = np.zeros(n, np.int32)
        if self.L.g5b_engine_decode_greedy(self.handle, first, n, out.ctypes.data) != 0:
            self._err("decode_greedy")
        return out

    def decode_speculative(self, first: int, n: int):
        """Greedy decode with the MTP layer's drafts verified two positions per pass.
        Returns (tokens, {"drafts", "accepted", "passes"})."""
        fn = self.L.g5b_engine_decode_speculative
        fn.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        out = np.zeros(n, np.int32)
        st = (C.c_long * 3)()
        if fn(self.handle, first, n, out.ctypes.data, st) != 0:
            self._err("decode_speculative")
        return out, {"drafts": int(st[0]), "accepted": int(st[1]), "passes": int(st[2])}

    def decode_sampled(self, first: int, n: int, temperature: float, top_p: float, seed: int):
        out = np.zeros(n, np.int32)
        if self.L.g5b_engine_decode_sampled(self.handle, first, n, C.c_float(temperature), C.c_float(top_p), seed,
                                            out.ctypes.data) != 0:
            self._err("decode_sampled")
        return out

    def sync(self):
        if self.L.g5b_engine_sync(self.handle) != 0:
            self._err("sync")

    def close(self):
        if getattr(self, "handle", None):
            self.L.g5b_engine_free(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def sample_host(logits, temperature: float, top_p: float, seed: int, step: int, device: int = 0) -> int:
    """One draw of the device sampler from host logits (g5b_sample_host)."""
    lg = _f32(logits).ravel()
    tok = C.c_int(-1)
    if lib().g5b_sample_host(lg.ctypes.data, lg.size, C.c_float(temperature), C.c_float(top_p), seed, step,
                             C.addressof(tok), device) != 0:
        raise RuntimeError("g5b_sample_host failed: " + (lib().g5b_last_error() or b"").decode())
    return tok.value
