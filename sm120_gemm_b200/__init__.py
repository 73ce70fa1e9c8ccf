"""B200 (sm_100a) GEMM plugins behind the reference project's registry / cache / dispatch API.

This Python package is a thin ctypes face over the C ABI in ``include/sm100_gemm.h`` so that
tests and the benchmark can drive the plugins; the C++ equivalent is ``csrc/gemm_config.h``.
It mirrors the reference's host interface by name (src/gemm_config.h): ``GemmConfig``
(:24-55), ``KernelRegistry`` (:65-120), ``AutotuneCache`` (:124-170), ``dispatch`` (:173-178).

There is no CPU fallback: every compute call goes to a CUDA kernel in a plugin, and a missing
plugin is an error.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass

from .gen_configs import DT_IDS, GemmConfig, generate_configs, heuristic_config, heuristic_ms

KERNEL_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "kernels")

GEMM_OK = 0
ACT_NONE, ACT_RELU, ACT_GELU, ACT_SILU = 0, 1, 2, 3       # GEMM_ACT_* of include/sm100_gemm.h
Y_BF16, Y_E4M3 = 0, 1                                     # GEMM_Y_*
ERROR_NAMES = {0: "GEMM_OK", 1: "GEMM_ERR_SHAPE", 2: "GEMM_ERR_CUDA", 3: "GEMM_ERR_DRIVER", 4: "GEMM_ERR_WORKSPACE",
               5: "GEMM_ERR_DEVICE_TIMEOUT", 6: "GEMM_ERR_ARG"}

# every symbol include/sm100_gemm.h declares
ABI_SYMBOLS = ("gemm_run", "gemm_run_ex", "gemm_config_name", "gemm_workspace_bytes", "gemm_can_run", "gemm_smem_bytes",
               "gemm_last_error", "gemm_last_error_message", "gemm_check_status", "gemm_run_no_alloc")
NO_ALLOC_SCRATCH_BYTES = 16 << 20  # GEMM_NO_ALLOC_SCRATCH_BYTES of include/sm100_gemm.h


class GemmError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"{ERROR_NAMES.get(code, code)}: {msg}")
        self.code = code


class GemmArgs(ctypes.Structure):
    """``struct GemmArgs`` of include/sm100_gemm.h."""

    _fields_ = [
        ("struct_size", ctypes.c_uint32), ("dtype", ctypes.c_uint32),
        ("M", ctypes.c_int32), ("N", ctypes.c_int32), ("K", ctypes.c_int32), ("group_size", ctypes.c_int32),
        ("X", ctypes.c_void_p), ("W", ctypes.c_void_p), ("Y", ctypes.c_void_p),
        ("x_scale", ctypes.c_void_p), ("w_scale", ctypes.c_void_p),
        ("x_scale_f", ctypes.c_float), ("w_scale_f", ctypes.c_float),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_size_t),
        ("sm_limit", ctypes.c_int32), ("reserved", ctypes.c_int32),
        ("stream", ctypes.c_void_p),
        ("y_num_peers", ctypes.c_int32), ("y_col_offset", ctypes.c_int32), ("y_ld", ctypes.c_int64),
        ("y_peers", ctypes.c_void_p * 8), ("y_multicast", ctypes.c_void_p),
        ("C", ctypes.c_void_p), ("bias", ctypes.c_void_p), ("alpha", ctypes.c_float), ("beta", ctypes.c_float),
        ("activation", ctypes.c_int32), ("y_dtype", ctypes.c_int32), ("y_scale", ctypes.c_float), ("amax", ctypes.c_void_p),
        ("y_forward", ctypes.c_int32),
    ]

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        if "alpha" not in kw:
            self.alpha = 1.0      # a plain GEMM; only the fused-epilogue plugins (e2) read it
        if "y_scale" not in kw:
            self.y_scale = 1.0


class GemmWeightFileInfo(ctypes.Structure):
    """``struct GemmWeightFileInfo`` of include/sm100_gemm_util.h (the first bytes of a weight file)."""

    _fields_ = [("magic", ctypes.c_char * 8), ("version", ctypes.c_uint32), ("dtype", ctypes.c_uint32), ("layout", ctypes.c_uint32),
                ("group", ctypes.c_uint32), ("N", ctypes.c_uint64), ("K", ctypes.c_uint64), ("elem_bytes", ctypes.c_uint64),
                ("scale_bytes", ctypes.c_uint64), ("tensor_scale", ctypes.c_float), ("checksum", ctypes.c_uint32)]


# every symbol include/sm100_gemm_util.h declares
UTIL_SYMBOLS = ("gemm_interleave_blocks", "gemm_spacer", "gemm_mx_tiled_scale_bytes", "gemm_mx_scales_to_tiled",
                "gemm_quant_e4m3_per_tensor", "gemm_quant_mx", "gemm_quant_int4_g128", "gemm_packed_weight_bytes",
                "gemm_packed_scale_bytes", "gemm_pack_int4_host", "gemm_unpack_int4_host", "gemm_pack_fp4_host", "gemm_unpack_fp4_host",
                "gemm_mx_scales_to_tiled_host", "gemm_mx_scales_from_tiled_host", "gemm_weight_file_write", "gemm_weight_file_info",
                "gemm_weight_file_read")


@dataclass
class LoadedKernel:
    """One dlopen'ed plugin (reference: struct LoadedKernel, src/gemm_config.h:58-62)."""

    config: GemmConfig
    lib: ctypes.CDLL
    path: str

    def can_run(self, M: int, N: int, K: int) -> bool:
        return bool(self.lib.gemm_can_run(M, N, K))

    def workspace_bytes(self, M: int, N: int, K: int) -> int:
        return int(self.lib.gemm_workspace_bytes(M, N, K))

    def smem_bytes(self) -> int:
        return int(self.lib.gemm_smem_bytes())

    def last_error(self) -> tuple[int, str]:
        return int(self.lib.gemm_last_error()), self.lib.gemm_last_error_message().decode()

    def check_status(self) -> None:
        rc = self.lib.gemm_check_status()
        if rc != GEMM_OK:
            raise GemmError(rc, self.last_error()[1])


def _bind(lib: ctypes.CDLL) -> None:
    vp, i32 = ctypes.c_void_p, ctypes.c_int
    lib.gemm_run.argtypes = [i32, i32, i32, vp, vp, vp, vp, vp]
    lib.gemm_run.restype = None
    lib.gemm_run_ex.argtypes = [ctypes.POINTER(GemmArgs)]
    lib.gemm_run_ex.restype = i32
    lib.gemm_config_name.restype = ctypes.c_char_p
    lib.gemm_workspace_bytes.argtypes = [i32, i32, i32]
    lib.gemm_workspace_bytes.restype = ctypes.c_size_t
    lib.gemm_can_run.argtypes = [i32, i32, i32]
    lib.gemm_can_run.restype = i32
    lib.gemm_smem_bytes.restype = ctypes.c_size_t
    lib.gemm_last_error.restype = i32
    lib.gemm_last_error_message.restype = ctypes.c_char_p
    lib.gemm_check_status.restype = i32
    lib.gemm_run_no_alloc.argtypes = [i32, i32, i32, vp, vp, vp, vp]
    lib.gemm_run_no_alloc.restype = i32


def load_plugin(path: str) -> LoadedKernel:
    stem = os.path.basename(path)
    if not (stem.startswith("libgemm_") and stem.endswith(".so")):
        raise ValueError(f"not a kernel plugin name: {path}")
    cfg = GemmConfig.parse(stem[len("libgemm_"):-3])
    if cfg is None:
        raise ValueError(f"cannot parse configuration from {stem}")
    lib = ctypes.CDLL(path)
    for sym in ABI_SYMBOLS:
        getattr(lib, sym)  # AttributeError if the plugin does not export the full ABI
    _bind(lib)
    if lib.gemm_config_name().decode() != cfg.name():
        raise ValueError(f"{stem}: file name and compiled-in configuration differ")
    return LoadedKernel(cfg, lib, path)


class KernelRegistry:
    """Scans a directory for ``libgemm_<config>.so`` (reference: src/gemm_config.h:65-120)."""

    def __init__(self) -> None:
        self.kernels: list[LoadedKernel] = []

    def load_dir(self, directory: str = KERNEL_DIR, dt: str | None = None) -> bool:
        if not os.path.isdir(directory):
            print(f"KernelRegistry: not a directory: {directory}")
            return False
        for f in sorted(os.listdir(directory)):
            if not (f.startswith("libgemm_") and f.endswith(".so")):
                continue
            cfg = GemmConfig.parse(f[len("libgemm_"):-3])
            if cfg is None:
                print(f"KernelRegistry: cannot parse config from {f}")
                continue
            if dt is not None and cfg.dt != dt:
                continue
            try:
                self.kernels.append(load_plugin(os.path.join(directory, f)))
            except (OSError, AttributeError, ValueError) as e:
                print(f"KernelRegistry: cannot load {f}: {e}")
        return bool(self.kernels)

    def get_valid(self, M: int, N: int, K: int, max_smem: int = 0, dt: str = "bf16") -> list[LoadedKernel]:
        out = []
        for k in self.kernels:
            if k.config.dt != dt or not k.config.is_valid_for(M, N, K):
                continue
            if max_smem > 0 and k.config.smem_bytes() > max_smem:
                continue
            out.append(k)
        return out

    def find(self, name: str) -> LoadedKernel | None:
        for k in self.kernels:
            if k.config.name() == name:
                return k
        return None

    def heuristic(self, M: int, N: int, K: int, dt: str = "bf16") -> LoadedKernel | None:
        """The loaded plugin with the smallest modelled time for the shape (no measurement, no cache)."""
        c = heuristic_config([k.config for k in self.kernels], dt, M, N, K)
        return self.find(c.name()) if c else None

    def select(self, cache: "AutotuneCache", M: int, N: int, K: int, dt: str = "bf16", gpus: int = 1) -> LoadedKernel | None:
        """Dispatch without autotuning: the cache entry when there is one (and its plugin is loaded), else the heuristic pick."""
        hit = cache.lookup(M, N, K, dt, gpus)
        k = self.find(hit[0].name()) if hit else None
        return k or self.heuristic(M, N, K, dt)


class AutotuneCache:
    """Text cache ``dt,g,M,N,K name ms`` (reference format ``M,N,K name ms``, src/gemm_config.h:122-170;
    three-field keys are still read, as bf16 on one GPU)."""

    def __init__(self) -> None:
        self.entries: dict[tuple, tuple[GemmConfig, float]] = {}

    def load(self, path: str) -> bool:
        if not os.path.exists(path):
            return False
        with open(path) as f:
            for line in f:
                line = line.strip()
                if not line or line.startswith("#"):
                    continue
                parts = line.split()
                if len(parts) != 3:
                    continue
                key = parts[0].split(",")
                cfg = GemmConfig.parse(parts[1])
                try:
                    ms = float(parts[2])
                    if len(key) == 3:
                        k = ("bf16", 1, int(key[0]), int(key[1]), int(key[2]))
                    elif len(key) == 5:
                        k = (key[0], int(key[1]), int(key[2]), int(key[3]), int(key[4]))
                    else:
                        continue
                except ValueError:
                    continue
                if cfg is not None:
                    self.entries[k] = (cfg, ms)
        return True

    def save(self, path: str) -> None:
        tmp = path + ".tmp"
        with open(tmp, "w") as f:
            f.write("# Autotune cache -- dt,gpus,M,N,K config_name time_ms\n")
            for (dt, g, M, N, K), (cfg, ms) in sorted(self.entries.items()):
                f.write(f"{dt},{g},{M},{N},{K} {cfg.name()} {ms:.6g}\n")
        os.replace(tmp, path)

    def lookup(self, M: int, N: int, K: int, dt: str = "bf16", gpus: int = 1):
        return self.entries.get((dt, gpus, M, N, K))

    def store(self, M: int, N: int, K: int, config: GemmConfig, time_ms: float, dt: str = "bf16", gpus: int = 1) -> None:
        self.entries[(dt, gpus, M, N, K)] = (config, time_ms)


def dispatch(kernel: LoadedKernel, M: int, N: int, K: int, X: int, W: int, Y: int, workspace: int = 0, stream: int = 0) -> None:
    """``kernel.fn(M,N,K,X,W,Y,workspace,stream)`` with raw device addresses (reference:
    dispatch, src/gemm_config.h:173-178).  Raises GemmError instead of the reference's exit()."""
    kernel.lib.gemm_run(M, N, K, X, W, Y, workspace, stream)
    code, msg = kernel.last_error()
    if code != GEMM_OK:
        raise GemmError(code, msg)


def dispatch_ex(kernel: LoadedKernel, args: GemmArgs) -> None:
    args.struct_size = ctypes.sizeof(GemmArgs)
    args.dtype = DT_IDS[kernel.config.dt]
    rc = kernel.lib.gemm_run_ex(ctypes.byref(args))
    if rc != GEMM_OK:
        raise GemmError(rc, kernel.last_error()[1])


_UTIL = None


def util_lib() -> ctypes.CDLL:
    """``libsm100gemm_util.so``: gemm_interleave_blocks, gemm_spacer, gemm_mx_scales_to_tiled (csrc/gemm_util.cu)."""
    global _UTIL
    if _UTIL is None:
        path = os.path.join(KERNEL_DIR, "libsm100gemm_util.so")
        if not os.path.exists(path):
            raise FileNotFoundError(f"{path} is missing: run __graft_entry__.build() or python -m sm120_gemm_b200.build")
        lib = ctypes.CDLL(path)
        lib.gemm_interleave_blocks.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_int,
                                               ctypes.c_int, ctypes.c_void_p]
        lib.gemm_interleave_blocks.restype = ctypes.c_int
        lib.gemm_spacer.argtypes = [ctypes.c_uint, ctypes.c_void_p]
        lib.gemm_spacer.restype = ctypes.c_int
        lib.gemm_mx_tiled_scale_bytes.argtypes = [ctypes.c_longlong, ctypes.c_int]
        lib.gemm_mx_tiled_scale_bytes.restype = ctypes.c_size_t
        lib.gemm_mx_scales_to_tiled.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p]
        lib.gemm_mx_scales_to_tiled.restype = ctypes.c_int
        vp, ll, ci = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int
        lib.gemm_quant_e4m3_per_tensor.argtypes = [vp, vp, vp, vp, ll, vp]
        lib.gemm_quant_mx.argtypes = [vp, vp, vp, ll, ci, ci, vp]
        lib.gemm_quant_int4_g128.argtypes = [vp, vp, vp, ll, ci, vp]
        for name in ("gemm_packed_weight_bytes", "gemm_packed_scale_bytes"):
            getattr(lib, name).argtypes = [ci, ll, ci]
            getattr(lib, name).restype = ctypes.c_size_t
        for name in ("gemm_pack_int4_host", "gemm_unpack_int4_host", "gemm_pack_fp4_host", "gemm_unpack_fp4_host",
                     "gemm_mx_scales_to_tiled_host", "gemm_mx_scales_from_tiled_host"):
            getattr(lib, name).argtypes = [vp, ll, ci, vp]
        lib.gemm_weight_file_write.argtypes = [ctypes.c_char_p, ci, ll, ci, ctypes.c_float, vp, vp]
        lib.gemm_weight_file_info.argtypes = [ctypes.c_char_p, ctypes.POINTER(GemmWeightFileInfo)]
        lib.gemm_weight_file_read.argtypes = [ctypes.c_char_p, vp, ctypes.c_size_t, vp, ctypes.c_size_t]
        _UTIL = lib
    return _UTIL


__all__ = ["heuristic_config", "heuristic_ms", "GemmWeightFileInfo", "UTIL_SYMBOLS", "util_lib", "GemmConfig", "generate_configs", "KernelRegistry", "AutotuneCache", "LoadedKernel", "GemmArgs", "GemmError",
           "dispatch", "dispatch_ex", "load_plugin", "KERNEL_DIR", "ABI_SYMBOLS"]
