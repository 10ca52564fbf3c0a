"""ctypes binding of libroller_b200.so (declared in include/roller_b200.h).

This is the only route from Python to the sm_100a kernels. There is no CPU fallback: when the
shared library is missing or cannot be loaded, `load()` raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libroller_b200.so"

MODE_1XTF32 = 1
MODE_3XTF32 = 3
MODE_BF16 = 16      # bf16 A and B, fp32 accumulation and C
MODE_F16 = 17       # fp16 A and B, fp32 accumulation and C
MODES_16BIT = (MODE_BF16, MODE_F16)
FLAG_ACCUMULATE = 1
FLAG_B_TRANSPOSED = 2
FLAG_C_16BIT = 4    # 16-bit modes only: C is written in the operand type instead of fp32
LAYOUT_GENERAL = 0
LAYOUT_SKINNY = 2
LAYOUT_CUDA_CORES = 3   # plain fp32 FMAs for a C of at most 16 rows per pass (3xTF32-class only)
# roller_b200_gemm_set_option
OPT_WAIT_LIMIT_CYCLES = 1
OPT_OVERLAP_LAUNCH = 2
OPT_TMA_STORE = 3
OPT_PROGRESSIVE_ROUNDS = 4
OPT_TEST_DROP_PUBLISH = 5
OPT_COOPERATIVE_FIXUP = 6
OPT_ROUND_RATIO = 7
OPT_EARLY_EXIT = 8
MAX_ROUNDS = 16
MAX_FLAG_TARGETS = 32
# device status words (what a bounded wait that ran out records)
DEV_TIMEOUT_FIXUP = 7
DEV_TIMEOUT_SLOT = 8
DEV_TIMEOUT_PEER = 9

OK = 0
ERR_INVALID = -1
ERR_UNSUPPORTED = -2
ERR_CUDA = -3
ERR_DEVICE = -4
ERR_TIMEOUT = -5
ERR_NOMEM = -6
ERR_TOO_LARGE = -7


class DevInfo(C.Structure):
    _fields_ = [
        ("cc_major", C.c_int), ("cc_minor", C.c_int),
        ("sm_count", C.c_int),
        ("smem_per_block_optin", C.c_int),
        ("smem_per_sm", C.c_int),
        ("regs_per_sm", C.c_int),
        ("l2_bytes", C.c_int),
        ("sm_clock_khz", C.c_int),
        ("mem_clock_khz", C.c_int),
        ("mem_bus_bits", C.c_int),
        ("tmem_columns", C.c_int),
        ("total_mem", C.c_size_t),
        ("name", C.c_char * 128),
    ]


class KTile(C.Structure):
    _fields_ = [
        ("block_m", C.c_int), ("block_n", C.c_int), ("rstep", C.c_int), ("cta_group", C.c_int),
        ("stages_1x", C.c_int), ("stages_3x", C.c_int),
        ("smem_1x", C.c_int), ("smem_3x", C.c_int),
        ("tmem_cols", C.c_int),
        ("threads_1x", C.c_int), ("threads_3x", C.c_int),
        ("layout", C.c_int),
        ("rstep_16", C.c_int), ("stages_16", C.c_int), ("smem_16", C.c_int),
    ]

    def as_dict(self) -> dict:
        return {name: getattr(self, name) for name, _ in self._fields_}


# name -> (restype, argtypes); every symbol include/roller_b200.h declares.
SIGNATURES = {
    "roller_b200_device_info": (C.c_int, [C.c_int, C.POINTER(DevInfo)]),
    "roller_b200_kernel_count": (C.c_int, []),
    "roller_b200_kernel_desc": (C.c_int, [C.c_int, C.POINTER(KTile)]),
    "roller_b200_gemm_create": (C.c_int, [C.POINTER(KTile), C.c_int, C.c_int, C.c_int, C.c_int,
                                          C.c_int, C.c_int, C.c_int, C.c_int,
                                          C.POINTER(C.c_void_p)]),
    "roller_b200_gemm_run": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "roller_b200_copy_block_async": (C.c_int, [C.c_void_p, C.c_longlong, C.c_void_p, C.c_longlong,
                                               C.c_longlong, C.c_longlong, C.c_void_p]),
    "roller_b200_gemm_time": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                        C.c_int, C.c_int, C.POINTER(C.c_float)]),
    "roller_b200_gemm_host": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "roller_b200_gemm_host_async": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                              C.c_void_p]),
    "roller_b200_gemm_launch_info": (C.c_int, [C.c_void_p] + [C.POINTER(C.c_int)] * 6),
    "roller_b200_gemm_schedule_info": (C.c_int, [C.c_void_p] + [C.POINTER(C.c_int)] * 4),
    "roller_b200_gemm_round_tiles": (C.c_int, [C.c_void_p, C.POINTER(C.c_int), C.c_int]),
    "roller_b200_gemm_set_chunk": (C.c_int, [C.c_void_p, C.c_int]),
    "roller_b200_gemm_set_grid": (C.c_int, [C.c_void_p, C.c_int]),
    "roller_b200_gemm_set_stream_k": (C.c_int, [C.c_void_p, C.c_int]),
    "roller_b200_gemm_set_option": (C.c_int, [C.c_void_p, C.c_int, C.c_longlong]),
    "roller_b200_gemm_run_synced": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                              C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32,
                                              C.c_void_p]),
    "roller_b200_flag_signal_async": (C.c_int, [C.POINTER(C.c_void_p), C.c_int, C.c_uint32,
                                                C.c_void_p]),
    "roller_b200_flag_wait_async": (C.c_int, [C.c_void_p, C.c_int, C.c_ulonglong, C.c_uint32,
                                              C.c_longlong, C.c_void_p, C.c_void_p]),
    "roller_b200_gemm_static_scratch": (C.c_int, [C.POINTER(KTile), C.c_int, C.c_int, C.c_int,
                                                  C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                                  C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "roller_b200_last_status": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint32)]),
    "roller_b200_gemm_destroy": (C.c_int, [C.c_void_p]),
    "roller_b200_strerror": (C.c_char_p, [C.c_int]),
    "roller_b200_last_cuda_error": (C.c_char_p, []),
}

_lib = None


def load() -> C.CDLL:
    """Load the shared library and type its entry points. Raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m mlir_roller_b200.build` "
            "(there is no CPU fallback for the GEMM path)")
    lib = C.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = header and library disagree
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


class RollerError(RuntimeError):
    """Raised for a non-zero roller_status; `.status` holds the code."""

    def __init__(self, status: int, where: str):
        lib = load()
        msg = lib.roller_b200_strerror(status).decode()
        if status == ERR_CUDA:
            msg += " (" + lib.roller_b200_last_cuda_error().decode() + ")"
        super().__init__(f"{where}: {msg} [status {status}]")
        self.status = status


def check(status: int, where: str) -> None:
    if status != OK:
        raise RollerError(status, where)


def device_info(dev: int = 0) -> DevInfo:
    info = DevInfo()
    check(load().roller_b200_device_info(dev, C.byref(info)), "roller_b200_device_info")
    return info


def kernel_tiles() -> list[KTile]:
    """The rTiles that have a compiled kernel."""
    lib = load()
    out = []
    for i in range(lib.roller_b200_kernel_count()):
        kt = KTile()
        check(lib.roller_b200_kernel_desc(i, C.byref(kt)), "roller_b200_kernel_desc")
        out.append(kt)
    return out


def find_tile(block_m: int, block_n: int, cta_group: int | None = None,
              layout: int = LAYOUT_GENERAL) -> KTile:
    for kt in kernel_tiles():
        if kt.block_m == block_m and kt.block_n == block_n and kt.layout == layout and \
                (cta_group is None or kt.cta_group == cta_group):
            return kt
    raise RollerError(ERR_UNSUPPORTED, f"find_tile({block_m}, {block_n}, {cta_group}, {layout})")


def _stream_ptr(stream) -> C.c_void_p:
    if stream is None:
        import torch
        stream = torch.cuda.current_stream()
    return C.c_void_p(getattr(stream, "cuda_stream", stream))


def gemm_static_scratch(tile: KTile, mode: int, M: int, N: int, K: int, lda: int, ldb: int,
                        ldc: int, a_ptr: int, b_ptr: int, c_ptr: int, status_ptr: int = 0,
                        stream=None) -> None:
    """Enqueue C = A @ B through the entry point that allocates nothing (its scratch is a fixed
    32 MiB array inside the library; see include/roller_b200.h for who needs that and the limits)."""
    check(load().roller_b200_gemm_static_scratch(C.byref(tile), mode, M, N, K, lda, ldb, ldc,
                                                 a_ptr, b_ptr, c_ptr, status_ptr or None,
                                                 _stream_ptr(stream)),
          "roller_b200_gemm_static_scratch")


def copy_block_async(dst_ptr: int, dst_ld: int, src_ptr: int, src_ld: int, rows: int, cols: int,
                     stream=None) -> None:
    """Enqueue a copy-engine copy of a rows x cols fp32 block between two device matrices
    (either may be a peer GPU's mapped memory)."""
    check(load().roller_b200_copy_block_async(dst_ptr, dst_ld, src_ptr, src_ld, rows, cols,
                                              _stream_ptr(stream)),
          "roller_b200_copy_block_async")


def flag_signal_async(target_ptrs, value: int, stream=None) -> None:
    """Enqueue a store of `value` into every address of `target_ptrs` (device pointers, possibly
    other GPUs' mapped memory), behind the work already on `stream`."""
    arr = (C.c_void_p * len(target_ptrs))(*target_ptrs)
    check(load().roller_b200_flag_signal_async(arr, len(target_ptrs), value & 0xFFFFFFFF,
                                               _stream_ptr(stream)),
          "roller_b200_flag_signal_async")


def flag_wait_async(flags_ptr: int, n: int, mask: int, value: int, status_ptr: int,
                    limit_cycles: int = 0, stream=None) -> None:
    """Enqueue a bounded wait until the words `flags_ptr[i]` selected by `mask` have reached
    `value`; a wait that runs out stores a non-zero code into the device word at `status_ptr`."""
    check(load().roller_b200_flag_wait_async(flags_ptr, n, mask, value & 0xFFFFFFFF, limit_cycles,
                                             status_ptr, _stream_ptr(stream)),
          "roller_b200_flag_wait_async")


class GemmPlan:
    """One rTile bound to one problem shape (owns the C-side plan)."""

    def __init__(self, tile: KTile, M: int, N: int, K: int, *, lda: int | None = None,
                 ldb: int | None = None, ldc: int | None = None, mode: int = MODE_3XTF32,
                 flags: int = 0):
        self._lib = load()
        self._h = C.c_void_p()
        self.tile = tile
        self.M, self.N, self.K, self.mode = M, N, K, mode
        self.flags = flags
        self.lda = K if lda is None else lda
        self.ldb = (K if flags & FLAG_B_TRANSPOSED else N) if ldb is None else ldb
        self.ldc = N if ldc is None else ldc
        check(self._lib.roller_b200_gemm_create(C.byref(tile), M, N, K, self.lda, self.ldb,
                                                self.ldc, mode, flags, C.byref(self._h)),
              "roller_b200_gemm_create")

    # -- raw-pointer interface (ints as returned by tensor.data_ptr())
    def run_ptr(self, a_ptr: int, b_ptr: int, c_ptr: int, stream=None) -> None:
        check(self._lib.roller_b200_gemm_run(self._h, a_ptr, b_ptr, c_ptr, _stream_ptr(stream)),
              "roller_b200_gemm_run")

    def run_synced_ptr(self, a_ptr: int, b_ptr: int, c_ptr: int, *, go_ptr: int = 0,
                       go_value: int = 0, arrive_ptr: int = 0, arrive_value: int = 0,
                       stream=None) -> None:
        """`run_ptr` whose kernel itself waits for the word at `go_ptr` to reach `go_value`
        before its first store into C and stores `arrive_value` at `arrive_ptr` after its last
        (RollerError(ERR_UNSUPPORTED) when the plan does not use the TMA-store output path)."""
        check(self._lib.roller_b200_gemm_run_synced(
            self._h, a_ptr, b_ptr, c_ptr, go_ptr or None, go_value & 0xFFFFFFFF,
            arrive_ptr or None, arrive_value & 0xFFFFFFFF, _stream_ptr(stream)),
            "roller_b200_gemm_run_synced")

    def _check_dtypes(self, A, B, Cout) -> None:
        """A and B must hold the element type the plan's mode names, C fp32 -- or that type too
        for a plan made with FLAG_C_16BIT (the C side only sees pointers)."""
        import torch
        want = {MODE_BF16: torch.bfloat16, MODE_F16: torch.float16}.get(self.mode, torch.float32)
        c_want = want if self.flags & FLAG_C_16BIT else torch.float32
        for name, t, dt in (("A", A, want), ("B", B, want), ("C", Cout, c_want)):
            if getattr(t, "dtype", dt) != dt:
                raise TypeError(f"{name} is {t.dtype}, this plan (mode {self.mode}) needs {dt}")

    def run(self, A, B, Cout, stream=None) -> None:
        self._check_dtypes(A, B, Cout)
        self.run_ptr(A.data_ptr(), B.data_ptr(), Cout.data_ptr(), stream)

    def time(self, A, B, Cout, warmup: int = 3, iters: int = 20, stream=None) -> float:
        self._check_dtypes(A, B, Cout)
        ms = C.c_float()
        check(self._lib.roller_b200_gemm_time(self._h, A.data_ptr(), B.data_ptr(), Cout.data_ptr(),
                                              _stream_ptr(stream), warmup, iters, C.byref(ms)),
              "roller_b200_gemm_time")
        return float(ms.value)

    def run_host(self, hA, hB, hC, stream=None, wait: bool = True) -> None:
        """hA/hB/hC: contiguous host arrays of the plan's element type (C fp32) (numpy or pinned torch CPU tensors). With
        `wait=False` the upload, kernel and readback are only enqueued on `stream`."""
        def ptr(x):
            return x.ctypes.data if hasattr(x, "ctypes") else x.data_ptr()
        fn = self._lib.roller_b200_gemm_host if wait else self._lib.roller_b200_gemm_host_async
        check(fn(self._h, ptr(hA), ptr(hB), ptr(hC), _stream_ptr(stream)), "roller_b200_gemm_host")

    def set_chunk(self, k_elems: int) -> None:
        check(self._lib.roller_b200_gemm_set_chunk(self._h, k_elems), "roller_b200_gemm_set_chunk")

    def set_grid(self, ctas: int) -> None:
        check(self._lib.roller_b200_gemm_set_grid(self._h, ctas), "roller_b200_gemm_set_grid")

    def set_stream_k(self, mode: int) -> None:
        """-1 automatic, 0 off (bit-identical results across tiles and shardings), 1 on."""
        check(self._lib.roller_b200_gemm_set_stream_k(self._h, mode),
              "roller_b200_gemm_set_stream_k")

    def set_option(self, option: int, value: int) -> None:
        """One of the OPT_* options of roller_b200_gemm_set_option."""
        check(self._lib.roller_b200_gemm_set_option(self._h, option, value),
              "roller_b200_gemm_set_option")

    def launch_info(self) -> dict:
        vals = [C.c_int() for _ in range(6)]
        check(self._lib.roller_b200_gemm_launch_info(self._h, *[C.byref(v) for v in vals]),
              "roller_b200_gemm_launch_info")
        keys = ("grid", "block", "smem_bytes", "tiles_m", "tiles_n", "max_clusters")
        return {k: v.value for k, v in zip(keys, vals)}

    def schedule_info(self) -> dict:
        vals = [C.c_int() for _ in range(4)]
        check(self._lib.roller_b200_gemm_schedule_info(self._h, *[C.byref(v) for v in vals]),
              "roller_b200_gemm_schedule_info")
        return {k: v.value for k, v in zip(("sk_tiles", "rounds", "unit_kb", "chunk_kb"), vals)}

    def round_tiles(self) -> list:
        """First tile of every round of the progressive schedule, then the number of tiles cut
        along K: rounds + 1 values."""
        buf = (C.c_int * (MAX_ROUNDS + 1))()
        check(self._lib.roller_b200_gemm_round_tiles(self._h, buf, MAX_ROUNDS + 1),
              "roller_b200_gemm_round_tiles")
        return list(buf[: self.schedule_info()["rounds"] + 1])

    def device_status(self) -> int:
        """The plan's device status word (0 = every bounded wait completed). Synchronises the
        device; a non-zero word is cleared by the read, so the plan can be launched again."""
        st = C.c_uint32()
        rc = self._lib.roller_b200_last_status(self._h, C.byref(st))
        if rc not in (OK, ERR_TIMEOUT):
            check(rc, "roller_b200_last_status")
        return int(st.value)

    def check_status(self) -> None:
        st = self.device_status()
        if st != 0:
            raise RollerError(ERR_TIMEOUT, f"device status word = {st}")

    def destroy(self) -> None:
        if self._h:
            self._lib.roller_b200_gemm_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass
