"""Loader of libwein_b200.so.  There is no CPU fallback: a missing library is an error."""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# WEIN_B200_TRACE=1 loads the diagnostic twin built by `python -m inferulm_b200.build --trace` (kernel-start time stamps)
LIB_PATH = os.path.join(HERE, "libwein_b200_trace.so" if os.environ.get("WEIN_B200_TRACE") == "1" else "libwein_b200.so")


class LibraryMissing(RuntimeError):
    pass


class WeinB200Error(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"wein_b200 status {code}: {msg}")
        self.code = code


_lib = None


def load():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise LibraryMissing(
                f"{LIB_PATH} not found: build it with `python -m inferulm_b200.build` (needs nvcc); "
                "there is no CPU or PyTorch fallback for these operators")
        try:
            import torch  # noqa: F401  (brings in the CUDA runtime / cuBLASLt the library links against)
        except Exception:
            pass
        _lib = C.CDLL(LIB_PATH)
        _lib.wein_b200_last_error.restype = C.c_char_p
        _lib.wein_b200_abi_version.restype = C.c_uint32
        if os.environ.get("WEIN_B200_GEMM_TUNE"):  # A/B switch "kw,ksplit,depth" (0 = automatic), see wein_b200_gemm_tune
            kw, ks, unr = (int(v) for v in os.environ["WEIN_B200_GEMM_TUNE"].split(","))
            _lib.wein_b200_gemm_tune(C.c_uint32(kw), C.c_uint32(ks), C.c_uint32(unr))
        if os.environ.get("WEIN_B200_PREFETCH_MB"):  # A/B switch: cap of the next-weights L2 prefetch (0 = off)
            _lib.wein_b200_gemm_prefetch_cap(C.c_uint64(int(os.environ["WEIN_B200_PREFETCH_MB"]) << 20))
        if os.environ.get("WEIN_B200_GEMM_IMPL"):  # A/B switch: 0 register-streaming, 1 bulk-copy staged skinny GEMM
            _lib.wein_b200_gemm_impl(C.c_uint32(int(os.environ["WEIN_B200_GEMM_IMPL"])))
        if os.environ.get("WEIN_B200_CARVEOUT"):  # A/B switch: shared-memory carve-out preference (percent, -1 = driver default)
            _lib.wein_b200_set_carveout(C.c_int32(int(os.environ["WEIN_B200_CARVEOUT"])))
        if os.environ.get("WEIN_B200_LT_TUNE"):  # A/B switch: 0 = keep cuBLASLt's first heuristic answer for forwards of > 32 rows
            _lib.wein_b200_gemm_lt_tune(C.c_uint32(int(os.environ["WEIN_B200_LT_TUNE"])))
        if os.environ.get("WEIN_B200_LITE"):  # A/B switch: 0 = a DeltaNet state snapshot per verify position instead of update records
            _lib.wein_b200_engine_lite(C.c_uint32(int(os.environ["WEIN_B200_LITE"])))
        if os.environ.get("WEIN_B200_FAST_SAMPLED"):  # A/B switch: 0 = sampled rounds keep the skinny GEMM up to 32 rows
            _lib.wein_b200_engine_fast_sampled(C.c_uint32(int(os.environ["WEIN_B200_FAST_SAMPLED"])))
        if os.environ.get("WEIN_B200_GDN_SPLIT"):  # A/B switch: 0 = one-launch DeltaNet layer at every batch size
            _lib.wein_b200_gdn_split(C.c_uint32(int(os.environ["WEIN_B200_GDN_SPLIT"])))
        if os.environ.get("WEIN_B200_PF_ROW_BYTES"):  # A/B switch: reach of the skinny GEMM's pre-wait L2 prefetch per weight row
            _lib.wein_b200_gemm_prefetch_row_bytes(C.c_uint32(int(os.environ["WEIN_B200_PF_ROW_BYTES"])))
        if os.environ.get("WEIN_B200_ABLATE"):  # profiling only: see wein_b200_engine_ablate
            _lib.wein_b200_engine_ablate(C.c_uint32(int(os.environ["WEIN_B200_ABLATE"])))
        if os.environ.get("WEIN_B200_PDL", "1") != "1":  # A/B switch: 0 = every kernel fully serialised, 3 = all but the GEMMs overlap
            _lib.wein_b200_set_pdl(C.c_uint32(int(os.environ["WEIN_B200_PDL"])))
    return _lib


def check(code):
    if code != 0:
        raise WeinB200Error(code, load().wein_b200_last_error().decode())
    return code
