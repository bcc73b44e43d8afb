"""ctypes bindings of the CPU checkers: the oracle restatement (oracle/_build) and, where it was
built, the unmodified reference (oracle/_ref).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by bench.py's CPU
baseline legs, never by the product package.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "_build", "libglm53f_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "libglm53f_ref.so")


def reference_tree() -> str:
    """Where the unmodified reference project lies: $GLM53F_REFERENCE, else a directory named
    `reference` beside this repository. It only has to exist where the checker is built."""
    return os.environ.get("GLM53F_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def build(reference_tree: str | None = None):
    """Compile the oracle, and the reference objects when the reference tree is present."""
    reference_tree = reference_tree or globals()["reference_tree"]()
    subprocess.run(["make", "-C", HERE, "oracle"], check=True, stdout=subprocess.DEVNULL)
    if os.path.isdir(os.path.join(reference_tree, "src", "core")):
        subprocess.run(["make", "-C", HERE, "ref", "ref-gpu-test", f"REF={reference_tree}"], check=True,
                       stdout=subprocess.DEVNULL)


def _pkg():
    mod = sys.modules.get("glm53f_b200")
    if mod is None:
        sys.path.insert(0, os.path.dirname(HERE))
        from __graft_entry__ import load_package
        mod = load_package()
    return mod


def _open(path, prefix):
    pkg = _pkg()
    L = C.CDLL(path)
    pkg._declare(L, prefix, C.c_void_p)
    create = getattr(L, f"{prefix}_model_create")
    create.restype = C.c_void_p
    create.argtypes = [C.POINTER(pkg.Config), C.c_char_p, C.c_char_p, C.c_int, C.c_int]
    return L


_libs = {}


def oracle_lib():
    if "orc" not in _libs:
        if not os.path.exists(ORACLE_SO):
            build()
        L = _open(ORACLE_SO, "orc")
        L.orc_synth_codes.argtypes = [C.c_void_p, C.c_uint64, C.c_int, C.c_int, C.c_int, C.c_size_t]
        L.orc_synth_codes.restype = None
        L.orc_synth_matrix_codes.argtypes = [C.c_void_p, C.c_uint64, C.c_char_p, C.c_size_t]
        L.orc_synth_matrix_codes.restype = None
        L.orc_synth_matrix_bf16.argtypes = [C.c_void_p, C.c_uint64, C.c_char_p, C.c_float, C.c_size_t]
        L.orc_synth_matrix_bf16.restype = None
        _libs["orc"] = L
    return _libs["orc"]


def have_ref() -> bool:
    return os.path.exists(REF_SO)


def ref_lib():
    if "ref" not in _libs:
        L = _open(REF_SO, "ref")
        L.ref_open_dir.restype = C.c_void_p
        L.ref_open_dir.argtypes = [C.c_char_p, C.c_int, C.c_int]
        L.ref_model_vocab.argtypes = [C.c_void_p]
        _libs["ref"] = L
    return _libs["ref"]


def _model_class(prefix):
    pkg = _pkg()

    class CpuModel(pkg.FlatModel):
        model_word = "model"

        def __init__(self, cfg, is_mla, is_dense, cap, kv_mode=0, _handle=None):
            self.L = oracle_lib() if prefix == "orc" else ref_lib()
            self.prefix = prefix
            self.cfg = cfg.copy()
            self._rows = {}
            if _handle is not None:
                self.handle = _handle
                return
            self._ml = bytes(bytearray(int(v) for v in is_mla))
            self._dn = bytes(bytearray(int(v) for v in is_dense))
            self.handle = getattr(self.L, f"{prefix}_model_create")(C.byref(self.cfg), self._ml, self._dn,
                                                                   cap, kv_mode)
            if not self.handle:
                raise RuntimeError(f"{prefix}_model_create failed")

        def load(self, name, arr, dtype, scale=None):
            super().load(name, arr, dtype, scale)
            self._rows[name] = arr.shape[0]

        def close(self):
            if getattr(self, "handle", None):
                getattr(self.L, f"{prefix}_model_free")(self.handle)
                self.handle = None

        def __del__(self):
            try:
                self.close()
            except Exception:
                pass

    return CpuModel


def OracleModel(*a, **k):
    return _model_class("orc")(*a, **k)


def RefModel(*a, **k):
    return _model_class("ref")(*a, **k)


def ref_open_dir(directory: str, cfg, cap: int, kv_mode: int = 0):
    """The reference's own loader on a checkpoint directory (glm53f_model_open)."""
    h = ref_lib().ref_open_dir(directory.encode(), cap, kv_mode)
    if not h:
        raise RuntimeError("glm53f_model_open failed")
    return _model_class("ref")(cfg, None, None, cap, _handle=h)


def matvec_host(prefix, arr, dtype, scale, br, bc, x):
    """glm53f_mm / glm53f_mm_batch on a free-standing matrix through the oracle or the reference."""
    pkg = _pkg()
    L = oracle_lib() if prefix == "orc" else ref_lib()
    t, keep = pkg.as_tensor(arr, dtype, scale)
    x = np.ascontiguousarray(x, dtype=np.float32)
    T = x.shape[0] if x.ndim == 2 else 1
    y = np.zeros((T, arr.shape[0]), np.float32)
    rc = getattr(L, f"{prefix}_matvec_host")(C.byref(t), br, bc, x.ctypes.data, T, y.ctypes.data)
    assert rc == 0
    return y if x.ndim == 2 else y[0]


def synth_codes(seed, layer, expert, which, count) -> np.ndarray:
    out = np.zeros(count, np.uint8)
    oracle_lib().orc_synth_codes(out.ctypes.data, seed, layer, expert, which, count)
    return out


def synth_matrix_codes(seed, name: str, count) -> np.ndarray:
    """E4M3 codes of the named matrix as g5b_engine_fill_matrix generates them on the GPU."""
    out = np.zeros(count, np.uint8)
    oracle_lib().orc_synth_matrix_codes(out.ctypes.data, seed, name.encode(), count)
    return out


def synth_matrix_bf16(seed, name: str, mul: float, count) -> np.ndarray:
    """BF16 bits of the named matrix as g5b_engine_fill_matrix generates them on the GPU."""
    out = np.zeros(count, np.uint16)
    oracle_lib().orc_synth_matrix_bf16(out.ctypes.data, seed, name.encode(), C.c_float(mul), count)
    return out


def rmsnorm_host(prefix, x, w, eps) -> np.ndarray:
    """glm53f_rmsnorm over the rows of x through the oracle or the reference; w may be None."""
    L = oracle_lib() if prefix == "orc" else ref_lib()
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, n = (x.shape[0], x.shape[1]) if x.ndim == 2 else (1, x.size)
    wv = None if w is None else np.ascontiguousarray(w, dtype=np.float32)
    y = np.zeros_like(x)
    rc = getattr(L, f"{prefix}_rmsnorm_host")(y.ctypes.data, x.ctypes.data, None if wv is None else wv.ctypes.data,
                                             n, rows, C.c_float(eps))
    if rc != 0:
        raise RuntimeError(f"{prefix}_rmsnorm_host failed")
    return y
