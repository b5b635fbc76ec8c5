"""ctypes binding of libnvfp4_b200.so (the C ABI declared in include/nvfp4_b200.h).

There is no CPU path: if the library is missing this module raises, it never
falls back to another implementation.
"""
from __future__ import annotations

import ctypes
import pathlib

_PKG = pathlib.Path(__file__).resolve().parent
LIB_PATH = _PKG / "libnvfp4_b200.so"

VARIANT_MSE, VARIANT_WEIGHTED, VARIANT_AMAX = 0, 1, 2
DT_BF16, DT_F16, DT_F32 = 0, 1, 2
ERR_TOO_LARGE = -8

EXPORTS = (
    "nvfp4_quant_launch", "nvfp4_quant_launch_impl", "nvfp4_quant_fused_launch", "nvfp4_quant_chain_launch", "nvfp4_quant_fused_last_status",
    "nvfp4_global_scale_launch", "nvfp4_global_scale_launch_static", "nvfp4_global_scale_static_max_bytes",
    "nvfp4_channel_sqnorm_launch", "nvfp4_channel_sqnorm_launch_strided", "nvfp4_gemm_peak_probe", "nvfp4_gemm_set_wait_limit_ns", "nvfp4_quant_fused_set_wait_limit_ns",
    "nvfp4_gemm_launch", "nvfp4_gemm_workspace_bytes", "nvfp4_gemm_prepare", "nvfp4_gemm_launch_prepared", "nvfp4_gemm_launch_grouped", "nvfp4_gemm_release", "nvfp4_gemm_last_status", "nvfp4_gemm_force_path", "nvfp4_gemm_tune", "nvfp4_gemm_tune_raster", "nvfp4_gemm_tune_pdl", "nvfp4_gemm_plan",
    "nvfp4_status_string", "nvfp4_abi_version", "nvfp4_stream_capture_id",
)

_lib = None


class Nvfp4Error(RuntimeError):
    """A launch was rejected or failed; `.status` holds the C ABI status code."""

    def __init__(self, status: int, what: str):
        super().__init__(f"{what}: {status_string(status)} (status {status})")
        self.status = status


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m nvfp4quant_test_b200.build` "
                "(needs nvcc; there is no CPU fallback)")
        L = ctypes.CDLL(str(LIB_PATH))
        i64, ci, vp, f32 = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_float
        L.nvfp4_quant_launch.restype = ci
        L.nvfp4_quant_launch.argtypes = [ci, vp, ci, vp, vp, vp, vp, i64, i64, i64, ci, ci, ci, vp]
        L.nvfp4_quant_launch_impl.restype = ci
        L.nvfp4_quant_launch_impl.argtypes = [ci, ci, vp, ci, vp, vp, vp, vp, i64, i64, i64, ci, ci, ci, vp]
        L.nvfp4_quant_fused_launch.restype = ci
        L.nvfp4_quant_fused_launch.argtypes = [ci, vp, ci, vp, f32, vp, vp, vp, vp, i64, i64, i64, ci, ci, ci, vp]
        L.nvfp4_quant_chain_launch.restype = ci
        L.nvfp4_quant_chain_launch.argtypes = [ci, vp, ci, vp, f32, vp, vp, vp, vp, i64, i64, i64, ci, ci, ci, vp]
        L.nvfp4_quant_fused_last_status.restype = ci
        L.nvfp4_quant_fused_last_status.argtypes = [vp, vp]
        L.nvfp4_global_scale_launch.restype = ci
        L.nvfp4_global_scale_launch.argtypes = [vp, ci, i64, f32, vp, vp, vp]
        L.nvfp4_global_scale_launch_static.restype = ci
        L.nvfp4_global_scale_launch_static.argtypes = [vp, ci, i64, f32, vp, vp]
        L.nvfp4_global_scale_static_max_bytes.restype = i64
        L.nvfp4_global_scale_static_max_bytes.argtypes = []
        L.nvfp4_gemm_peak_probe.restype = ci
        L.nvfp4_gemm_peak_probe.argtypes = [ci, ci, vp, vp]
        L.nvfp4_gemm_set_wait_limit_ns.restype = ci
        L.nvfp4_gemm_set_wait_limit_ns.argtypes = [ctypes.c_uint64]
        L.nvfp4_quant_fused_set_wait_limit_ns.restype = ci
        L.nvfp4_quant_fused_set_wait_limit_ns.argtypes = [ctypes.c_uint64]
        L.nvfp4_channel_sqnorm_launch.restype = ci
        L.nvfp4_channel_sqnorm_launch.argtypes = [vp, ci, i64, i64, vp, vp]
        L.nvfp4_channel_sqnorm_launch_strided.restype = ci
        L.nvfp4_channel_sqnorm_launch_strided.argtypes = [vp, ci, i64, i64, i64, vp, vp]
        L.nvfp4_gemm_launch.restype = ci
        L.nvfp4_gemm_launch.argtypes = [vp, vp, vp, vp, vp, vp, i64, i64, i64, vp, ctypes.c_size_t, vp]
        L.nvfp4_gemm_prepare.restype = ci
        L.nvfp4_gemm_prepare.argtypes = [vp, vp, i64, i64, vp]
        L.nvfp4_gemm_launch_prepared.restype = ci
        L.nvfp4_gemm_launch_prepared.argtypes = [vp, vp, vp, vp, vp, i64, vp, ctypes.c_size_t, vp]
        L.nvfp4_stream_capture_id.restype = ci
        L.nvfp4_stream_capture_id.argtypes = [vp, vp]
        L.nvfp4_gemm_launch_grouped.restype = ci
        L.nvfp4_gemm_launch_grouped.argtypes = [vp, ci, vp, vp, vp, vp, vp, i64, vp]
        L.nvfp4_gemm_release.restype = ci
        L.nvfp4_gemm_release.argtypes = [vp]
        L.nvfp4_gemm_workspace_bytes.restype = ctypes.c_size_t
        L.nvfp4_gemm_workspace_bytes.argtypes = [i64, i64, i64]
        L.nvfp4_gemm_last_status.restype = ci
        L.nvfp4_gemm_last_status.argtypes = [vp, vp]
        L.nvfp4_gemm_plan.restype = ci
        L.nvfp4_gemm_plan.argtypes = [i64, i64, i64, ci, vp, vp]
        L.nvfp4_gemm_tune_pdl.restype = ci
        L.nvfp4_gemm_tune_pdl.argtypes = [ci]
        L.nvfp4_gemm_tune_raster.restype = ci
        L.nvfp4_gemm_tune_raster.argtypes = [ci]
        L.nvfp4_gemm_tune.restype = ci
        L.nvfp4_gemm_tune.argtypes = [ci, ci]
        L.nvfp4_gemm_force_path.restype = ci
        L.nvfp4_gemm_force_path.argtypes = [ci]
        L.nvfp4_status_string.restype = ctypes.c_char_p
        L.nvfp4_status_string.argtypes = [ci]
        L.nvfp4_abi_version.restype = ci
        _lib = L
    return _lib


def status_string(status: int) -> str:
    return lib().nvfp4_status_string(int(status)).decode()


def check(status: int, what: str) -> None:
    if status != 0:
        raise Nvfp4Error(status, what)


def dtype_code(dtype) -> int:
    import torch

    try:
        return {torch.bfloat16: DT_BF16, torch.float16: DT_F16, torch.float32: DT_F32}[dtype]
    except KeyError:
        raise ValueError(f"input dtype must be bfloat16, float16 or float32, got {dtype}") from None


_raw_stream = None


def current_stream_ptr(device) -> int:
    """cudaStream_t of torch's current stream on `device`, as an integer."""
    global _raw_stream
    import torch

    if _raw_stream is None:
        # the accessor torch's own launchers use: ~0.2 us instead of ~2 us for building a Stream object
        _raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", False)
    if _raw_stream:
        index = device.index if isinstance(device, torch.device) else torch.device(device).index
        return _raw_stream(torch.cuda.current_device() if index is None else index)
    return torch.cuda.current_stream(device).cuda_stream


class _NoGuard:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_GUARD = _NoGuard()


def device_guard(device):
    """Context that makes `device` current for a launch; free when it already is (the usual case)."""
    import torch

    if device.index is None or device.index == torch.cuda.current_device():
        return _NO_GUARD
    return torch.cuda.device(device)


def capture_id(stream: int) -> int:
    """0 unless `stream` (a cudaStream_t as an integer) is being captured into a CUDA graph, else the capture's id."""
    out = ctypes.c_ulonglong(0)
    if lib().nvfp4_stream_capture_id(stream, ctypes.byref(out)) != 0:
        return 0
    return out.value


class StreamScratch:
    """Small zero-initialised device buffers keyed by (device, stream): launches on one stream may share a scratch
    (the kernels leave it zeroed), launches that may overlap need their own.  Holds at most `capacity` stream entries
    and drops the least recently used one beyond that, so a process that keeps creating streams does not grow it
    without bound (a dropped buffer goes back to torch's caching allocator, which only hands it out again in stream
    order).

    Launches recorded into a CUDA graph get a scratch per CAPTURE instead: graphs captured one after the other on the
    same stream may be replayed at the same time on different streams.  Those buffers are taken from a few zeroed
    spares that are set aside outside captures (a buffer created during a capture would add a fill node to the graph;
    that is what happens when the spares run out) and are kept for the life of the process, since a graph that uses
    one may be replayed at any time (8 or 16 bytes each)."""

    SPARES = 8

    def __init__(self, words: int, capacity: int = 32):
        from collections import OrderedDict

        self.words, self.capacity, self._d = words, capacity, OrderedDict()
        self._captures, self._spare = {}, {}

    def _zeros(self, device):
        import torch

        return torch.zeros(self.words, dtype=torch.int32, device=device)

    def get(self, device, stream: int):
        on_gpu = getattr(device, "type", "cpu") == "cuda"
        cap = capture_id(stream) if on_gpu else 0
        if cap:
            key = (device, cap, stream)      # a capture may span forked streams: one scratch per stream of it
            buf = self._captures.get(key)
            if buf is None:
                spare = self._spare.get(device)
                buf = self._captures[key] = spare.pop() if spare else self._zeros(device)
            return buf
        if on_gpu:
            spare = self._spare.setdefault(device, [])
            while len(spare) < self.SPARES:
                spare.append(self._zeros(device))
        key = (device, stream)
        buf = self._d.get(key)
        if buf is None:
            buf = self._d[key] = self._zeros(device)
            while len(self._d) > self.capacity:
                self._d.popitem(last=False)
        else:
            self._d.move_to_end(key)
        return buf

    def __len__(self):
        return len(self._d)
