"""ctypes binding of libvuib200 (include/vuib200.h) and its in-tree build.

There is no fallback: if the shared library is missing and cannot be built, or a
call returns a non-zero status, this module raises.
"""

from __future__ import annotations

import ctypes as C
import os
import shutil
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_HERE)
LIB_PATH = os.path.join(_HERE, "libvuib200.so")
_CSRC = os.path.join(_HERE, "csrc")
_OBJ = os.path.join(_CSRC, "_obj")
_API_H = os.path.join(_ROOT, "include", "vuib200.h")
# translation unit -> the headers it includes (a unit is recompiled when one of them changes)
UNITS = {
    "vuib200.cu": ["decode_kernels.cuh", "tc_gemm.cuh", "fused_blocks.cuh", "depth_group.cuh", "prefill_attn.cuh"],
    "codec.cu": ["codec_kernels.cuh"],
    "codec_enc.cu": ["codec_enc_kernels.cuh"],
}
SOURCES = [os.path.join(_CSRC, u) for u in UNITS]
HEADERS = sorted({os.path.join(_CSRC, h) for hs in UNITS.values() for h in hs}) + [_API_H]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]

VUIB_MAX_LAYERS = 64


class VuibConfig(C.Structure):
    _fields_ = [
        ("d_model", C.c_int32), ("n_layers", C.c_int32), ("n_heads", C.c_int32),
        ("n_kv_heads", C.c_int32), ("head_dim", C.c_int32), ("ffn", C.c_int32),
        ("n_quantizers", C.c_int32), ("codebook_size", C.c_int32),
        ("rq_d_model", C.c_int32), ("rq_n_layers", C.c_int32), ("rq_n_heads", C.c_int32),
        ("rq_ffn", C.c_int32),
        ("norm_eps", C.c_float), ("rq_norm_eps", C.c_float),
        ("n_slots", C.c_int32), ("max_seq", C.c_int32), ("max_rows", C.c_int32),
        ("max_prefill_rows", C.c_int32),
    ]


_PL = C.c_void_p * VUIB_MAX_LAYERS


class VuibWeights(C.Structure):
    _fields_ = [
        ("audio_emb", C.c_void_p), ("codec_head", C.c_void_p), ("eos_w", C.c_void_p),
        ("eos_b", C.c_void_p), ("final_norm", C.c_void_p),
        ("attn_norm", _PL), ("wqkv", _PL), ("out_proj", _PL), ("mlp_norm", _PL),
        ("w1", _PL), ("w3", _PL), ("w2", _PL),
        ("rq_backbone_proj", C.c_void_p), ("rq_code_emb", C.c_void_p), ("rq_pos_emb", C.c_void_p),
        ("rq_head", C.c_void_p), ("rq_norm", C.c_void_p),
        ("rq_attn_norm", _PL), ("rq_wqkv", _PL), ("rq_out_proj", _PL), ("rq_mlp_norm", _PL),
        ("rq_w1", _PL), ("rq_w3", _PL), ("rq_w2", _PL),
    ]


class VuibSampling(C.Structure):
    _fields_ = [
        ("temperature", C.c_float), ("top_k_cb0", C.c_int32), ("top_k_rq", C.c_int32),
        ("rep_penalty", C.c_float), ("rep_window", C.c_int32), ("n_codebooks", C.c_int32),
        ("seed", C.c_uint64),
    ]


VUIB_CODEC_LAYERS, VUIB_CODEC_STAGES, VUIB_CODEC_BLOCKS = 8, 2, 4
_F = C.c_void_p  # const float* on the device


class VuibCodecConfig(C.Structure):
    _fields_ = [
        ("n_q", C.c_int32), ("codebook_size", C.c_int32), ("codebook_dim", C.c_int32), ("vq_dim", C.c_int32),
        ("latent_dim", C.c_int32), ("d_model", C.c_int32), ("n_layers", C.c_int32), ("n_heads", C.c_int32),
        ("mlp_dim", C.c_int32), ("max_seq", C.c_int32), ("decoder_dim", C.c_int32),
        ("rates", C.c_int32 * VUIB_CODEC_BLOCKS), ("norm_eps", C.c_float),
    ]


class VuibSnakeW(C.Structure):
    _fields_ = [("ea", _F), ("ib", _F)]


class VuibConvW(C.Structure):
    _fields_ = [("w", _F), ("b", _F)]


class VuibCodecLayerW(C.Structure):
    _fields_ = [("ln1", _F), ("wqkv", _F), ("wo", _F), ("attn_scale", _F), ("ln2", _F), ("gate", _F), ("up", _F),
                ("down", _F), ("mlp_scale", _F)]


class VuibUpStageW(C.Structure):
    _fields_ = [("up", VuibConvW), ("dw", VuibConvW), ("ln_w", _F), ("ln_b", _F), ("pw1", VuibConvW),
                ("pw2", VuibConvW), ("gamma", _F)]


class VuibResUnitW(C.Structure):
    _fields_ = [("act1", VuibSnakeW), ("conv1", VuibConvW), ("act2", VuibSnakeW), ("conv2", VuibConvW)]


class VuibDecBlockW(C.Structure):
    _fields_ = [("act", VuibSnakeW), ("up", VuibConvW), ("res", VuibResUnitW * 3)]


class VuibCodecWeights(C.Structure):
    _fields_ = [
        ("codebook", _F * 16), ("sem_proj", _F), ("acq_proj", _F), ("pre_conv", VuibConvW), ("in_proj", VuibConvW),
        ("layer", VuibCodecLayerW * VUIB_CODEC_LAYERS), ("norm", _F), ("out_proj", VuibConvW),
        ("rope_cos", _F), ("rope_sin", _F), ("stage", VuibUpStageW * VUIB_CODEC_STAGES), ("dec_in", VuibConvW),
        ("block", VuibDecBlockW * VUIB_CODEC_BLOCKS), ("final_act", VuibSnakeW), ("final_conv", VuibConvW),
    ]


class VuibCodecEncConfig(C.Structure):
    _fields_ = [("base_dim", C.c_int32), ("ratios", C.c_int32 * 4), ("d_model", C.c_int32), ("n_layers", C.c_int32),
                ("n_heads", C.c_int32), ("mlp_dim", C.c_int32), ("max_samples", C.c_int32)]


class VuibEncResBlockW(C.Structure):
    _fields_ = [("c3", VuibConvW), ("c1", VuibConvW)]


class VuibEncLayerW(C.Structure):
    _fields_ = [(n, _F) for n in ("ln1_w", "ln1_b", "wqkv", "wo", "attn_scale", "ln2_w", "ln2_b", "fc1", "fc2", "mlp_scale")]


class VuibCodecEncWeights(C.Structure):
    _fields_ = [
        ("conv_in", VuibConvW), ("res", VuibEncResBlockW * 4), ("down", VuibConvW * 4), ("conv_out", VuibConvW),
        ("layer", VuibEncLayerW * VUIB_CODEC_LAYERS), ("rope_cos", _F), ("rope_sin", _F), ("downsample", _F),
        ("sem_in", _F), ("acq_in", _F), ("codebook", _F * 16), ("codebook_norm2", _F * 16),
    ]


# name -> (restype, argtypes); every symbol include/vuib200.h declares
_P = C.c_void_p
SYMBOLS = {
    "vuib_abi_version": (C.c_int32, []),
    "vuib_create": (C.c_int32, [C.POINTER(VuibConfig), C.POINTER(_P)]),
    "vuib_destroy": (C.c_int32, [_P]),
    "vuib_last_error": (C.c_int32, [_P, C.c_char_p, C.c_size_t]),
    "vuib_workspace_bytes": (C.c_int32, [_P, C.POINTER(C.c_size_t)]),
    "vuib_bind_workspace": (C.c_int32, [_P, _P, C.c_size_t]),
    "vuib_bind_weights": (C.c_int32, [_P, C.POINTER(VuibWeights)]),
    "vuib_bind_kv": (C.c_int32, [_P, C.POINTER(_P), C.POINTER(_P), _P]),
    "vuib_bind_rope": (C.c_int32, [_P, _P]),
    "vuib_set_sampling": (C.c_int32, [_P, C.POINTER(VuibSampling), _P]),
    "vuib_set_stats": (C.c_int32, [_P, _P]),
    "vuib_set_taps": (C.c_int32, [_P, _P, _P]),
    "vuib_prefill": (C.c_int32, [_P, C.c_int32, _P, _P, _P, _P, _P]),
    "vuib_backbone_step": (C.c_int32, [_P, C.c_int32, _P, _P, _P, _P, _P, _P, _P]),
    "vuib_heads": (C.c_int32, [_P, C.c_int32, _P, _P, _P, _P]),
    "vuib_depth_step": (C.c_int32, [_P, C.c_int32, _P, _P, _P, _P, C.c_int32, _P, _P, _P]),
    "vuib_decode_frame": (C.c_int32, [_P, C.c_int32, _P, _P, _P, _P, _P, _P, _P, _P]),
    "vuib_frame_host_capture": (C.c_int32, [_P, C.c_int32, C.c_int32, _P, _P, _P, _P, _P, _P, _P, _P]),
    "vuib_frame_host": (C.c_int32, [_P, C.c_int32, C.c_int32, _P, _P, _P, _P]),
    "vuib_attention": (C.c_int32, [_P, C.c_int32, C.c_int32, _P, _P, _P, _P, _P]),
    "vuib_attention_noalloc": (C.c_int32, [C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P, _P, _P, _P, _P, _P, _P,
                                           C.c_char_p, C.c_size_t]),
    "vuib_embed_codes": (C.c_int32, [_P, C.c_int32, _P, _P, _P]),
    "vuib_sample_rows": (C.c_int32, [_P, C.c_int32, _P, _P, C.c_int32, _P, _P]),
    "vuib_debug_norm_linear": (C.c_int32, [_P, C.c_int32, _P, _P, _P, C.c_int32, _P, C.c_int32, _P]),
    "vuib_debug_linear_rope": (C.c_int32, [_P, C.c_int32, _P, _P, _P, _P, C.c_int32, _P]),
    "vuib_rep_reset": (C.c_int32, [_P, C.c_int32, _P]),
    "vuib_rep_state": (C.c_int32, [_P, C.c_int32, _P, _P, _P]),
    "vuib_reset_state": (C.c_int32, [_P, _P]),
    "vuib_read_trace": (C.c_int32, [_P, C.POINTER(C.c_uint64), C.c_int32]),
    "vuib_set_wait_limit": (C.c_int32, [_P, C.c_uint32]),
    "vuib_debug_withhold_arrival": (C.c_int32, [_P, _P]),
    "vuib_set_seq_len": (C.c_int32, [_P, C.c_int32, C.c_int32]),
    "vuib_get_seq_len": (C.c_int32, [_P, C.c_int32, C.POINTER(C.c_int32)]),
    "vuib_check_device_flag": (C.c_int32, [_P, _P]),
    "vuib_launch_count": (C.c_int64, [_P]),
    "vuib_codec_create": (C.c_int32, [C.POINTER(VuibCodecConfig), C.POINTER(_P)]),
    "vuib_codec_destroy": (C.c_int32, [_P]),
    "vuib_codec_last_error": (C.c_int32, [_P, C.c_char_p, C.c_size_t]),
    "vuib_codec_workspace_bytes": (C.c_int32, [_P, C.POINTER(C.c_size_t)]),
    "vuib_codec_bind_workspace": (C.c_int32, [_P, _P, C.c_size_t]),
    "vuib_codec_bind_weights": (C.c_int32, [_P, C.POINTER(VuibCodecWeights)]),
    "vuib_codec_reset": (C.c_int32, [_P, _P]),
    "vuib_codec_decode_frame": (C.c_int32, [_P, _P, C.c_int32, _P, _P]),
    "vuib_codec_position": (C.c_int32, [_P, C.POINTER(C.c_int32), _P]),
    "vuib_codec_check_flag": (C.c_int32, [_P, _P]),
    "vuib_codec_read_tap": (C.c_int32, [_P, C.c_int32, C.POINTER(C.c_float), C.c_int32, _P]),
    "vuib_codec_launch_count": (C.c_int64, [_P]),
    "vuib_codec_enc_create": (C.c_int32, [C.POINTER(VuibCodecEncConfig), C.POINTER(_P)]),
    "vuib_codec_enc_destroy": (C.c_int32, [_P]),
    "vuib_codec_enc_last_error": (C.c_int32, [_P, C.c_char_p, C.c_size_t]),
    "vuib_codec_enc_workspace_bytes": (C.c_int32, [_P, C.POINTER(C.c_size_t)]),
    "vuib_codec_enc_bind_workspace": (C.c_int32, [_P, _P, C.c_size_t]),
    "vuib_codec_enc_bind_weights": (C.c_int32, [_P, C.POINTER(VuibCodecEncWeights)]),
    "vuib_codec_enc_encode": (C.c_int32, [_P, _P, C.c_int32, C.c_int32, _P, _P]),
    "vuib_codec_enc_read_latent": (C.c_int32, [_P, C.POINTER(C.c_float), C.c_int32, _P]),
    "vuib_codec_enc_launch_count": (C.c_int64, [_P]),
}


def _src_hash() -> str:
    import hashlib

    h = hashlib.sha256()
    for p in SOURCES + HEADERS:
        with open(p, "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _stale() -> bool:
    """True when the .so is missing or was built from other sources (a content
    hash beside the .so decides, not mtimes, which a copy of the tree changes)."""
    if not os.path.exists(LIB_PATH) or not os.path.exists(LIB_PATH + ".srchash"):
        return True
    with open(LIB_PATH + ".srchash") as f:
        return f.read().strip() != _src_hash()


def _unit_hash(unit: str) -> str:
    import hashlib

    h = hashlib.sha256()
    for p in [os.path.join(_CSRC, unit)] + [os.path.join(_CSRC, x) for x in UNITS[unit]] + [_API_H]:
        with open(p, "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _compile_unit(nvcc: str, unit: str, verbose: bool) -> str:
    """Compile one translation unit to an object file, unless an object of the same inputs exists."""
    obj = os.path.join(_OBJ, unit + ".o")
    stamp, want = obj + ".srchash", _unit_hash(unit)
    if os.path.exists(obj) and os.path.exists(stamp):
        with open(stamp) as f:
            if f.read().strip() == want:
                return obj
    cmd = [nvcc, *NVCC_FLAGS, "-c", "-o", obj, os.path.join(_CSRC, unit)]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {unit}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        print(res.stderr)
    with open(stamp, "w") as f:
        f.write(want)
    return obj


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile csrc/*.cu for sm_100a into vui_b200/libvuib200.so (in-tree): one object per
    translation unit, compiled side by side, then one link."""
    if not force and not _stale():
        return LIB_PATH
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("libvuib200.so is missing or stale and nvcc was not found to build it")
    os.makedirs(_OBJ, exist_ok=True)
    if force:
        for u in UNITS:
            if os.path.exists(os.path.join(_OBJ, u + ".o.srchash")):
                os.remove(os.path.join(_OBJ, u + ".o.srchash"))
    from concurrent.futures import ThreadPoolExecutor

    with ThreadPoolExecutor(max_workers=len(UNITS)) as pool:
        objs = list(pool.map(lambda u: _compile_unit(nvcc, u, verbose), UNITS))
    res = subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC", "-shared",
                          "-o", LIB_PATH, *objs], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc link failed:\n{res.stdout}\n{res.stderr}")
    with open(LIB_PATH + ".srchash", "w") as f:
        f.write(_src_hash())
    return LIB_PATH


_lib = None


def load() -> C.CDLL:
    """Load the library (building it when the sources are newer) and type every symbol."""
    global _lib
    if _lib is not None:
        return _lib
    if _stale() and (shutil.which("nvcc") or os.path.exists("/usr/local/cuda/bin/nvcc")):
        build_library()
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} not found: build it with `python -c 'import __graft_entry__ as g; g.build()'`"
        )
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)  # AttributeError if the export is missing
        fn.restype = res
        fn.argtypes = args
    if lib.vuib_abi_version() != 1:
        raise RuntimeError("libvuib200 ABI version mismatch")
    _lib = lib
    return lib


class VuibError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"libvuib200 status {code}: {msg}")
        self.code = code


def check(handle, code: int) -> None:
    if code == 0:
        return
    buf = C.create_string_buffer(256)
    if handle:
        load().vuib_last_error(handle, buf, 256)
    raise VuibError(code, buf.value.decode() or "(no message)")
