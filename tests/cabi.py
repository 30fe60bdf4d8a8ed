"""ctypes binding of include/efm_b200.h for the tests, smoke() and bench.py.

Loads the in-tree lib/libefm_b200.so; raises if it is missing (there is no fallback).  The
signatures below are checked against the header by tests/test_cabi_exports.py.
"""
from __future__ import annotations

import ctypes as C
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "edge-fm-x_b200")
LIB_PATH = os.path.join(PKG, "lib", "libefm_b200.so")
PY_DIR = os.path.join(PKG, "python")

EFM_OK = 0
EFM_F32, EFM_F16, EFM_BF16, EFM_I32 = 0, 1, 2, 3
EFM_MEM_HOST, EFM_MEM_DEVICE = 0, 1


class ModelDesc(C.Structure):
    _fields_ = [("struct_size", C.c_int32), ("num_layers", C.c_int32), ("hidden", C.c_int32),
                ("q_heads", C.c_int32), ("kv_heads", C.c_int32), ("head_dim", C.c_int32),
                ("intermediate", C.c_int32), ("vocab", C.c_int32), ("rms_eps", C.c_float),
                ("rope_theta", C.c_float), ("tied_lm_head", C.c_int32), ("use_mrope", C.c_int32),
                ("mrope_section", C.c_int32 * 3), ("max_prefill_tokens", C.c_int32),
                ("max_response_tokens", C.c_int32)]


class VitDesc(C.Structure):
    _fields_ = [("struct_size", C.c_int32), ("depth", C.c_int32), ("hidden", C.c_int32), ("heads", C.c_int32),
                ("intermediate", C.c_int32), ("out_hidden", C.c_int32), ("patch", C.c_int32),
                ("temporal_patch", C.c_int32), ("in_channels", C.c_int32), ("merge", C.c_int32),
                ("window", C.c_int32), ("n_fullatt", C.c_int32), ("fullatt", C.c_int32 * 8),
                ("rms_eps", C.c_float), ("rope_theta", C.c_float), ("max_patches", C.c_int32)]


class VlaDesc(C.Structure):
    _fields_ = [("struct_size", C.c_int32)] + [(n, C.c_int32) for n in (
        "image_size", "patch", "vit_layers", "vit_hidden", "vit_heads", "vit_mlp", "shuffle", "n_images", "hidden", "layers",
        "q_heads", "kv_heads", "head_dim", "mlp", "vocab", "lang_tokens", "expert_hidden", "expert_mlp", "state_dim",
        "action_dim", "chunk", "steps")] + [("rope_theta", C.c_float), ("rms_eps", C.c_float), ("ln_eps", C.c_float)]


class Sampling(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_p", C.c_float), ("top_k", C.c_int32),
                ("reserved", C.c_uint32), ("seed", C.c_uint64)]


P = C.c_void_p
I32 = C.c_int32
SIGNATURES = {
    "efm_b200_create": (I32, [C.POINTER(ModelDesc), I32, I32, I32, C.POINTER(P)]),
    "efm_b200_destroy": (I32, [P]),
    "efm_b200_last_error": (C.c_char_p, [P]),
    "efm_b200_version": (C.c_char_p, []),
    "efm_b200_tp_unique_id": (I32, [P]),
    "efm_b200_tp_init": (I32, [P, P]),
    "efm_b200_tp_peer_export": (I32, [P, P]),
    "efm_b200_tp_peer_import": (I32, [P, P, I32]),
    "efm_b200_tp_set_wait_limit": (I32, [P, C.c_int64, C.c_double]),
    "efm_b200_tp_host_wait": (I32, [P, C.CFUNCTYPE(C.c_int, P), P, C.c_double]),
    "efm_b200_set_weight": (I32, [P, C.c_char_p, P, C.POINTER(C.c_int64), I32, I32, I32]),
    "efm_b200_set_decode_weight": (I32, [P, C.c_char_p, P, C.POINTER(C.c_int64), I32, I32, I32]),
    "efm_b200_finalize_weights": (I32, [P]),
    "efm_b200_alloc_kv_slot": (I32, [P, I32, I32]),
    "efm_b200_kv_layer_ptr": (I32, [P, I32, I32, C.POINTER(P), C.POINTER(I32)]),
    "efm_b200_set_sampling": (I32, [P, C.POINTER(Sampling)]),
    "efm_b200_prefill": (I32, [P, I32, C.POINTER(I32), I32, I32, P, I32, I32, I32, C.POINTER(I32), I32]),
    "efm_b200_set_prefill_graph": (I32, [P, I32]),
    "efm_b200_prefill_graph_stats": (I32, [P, C.POINTER(I32), C.POINTER(C.c_int64)]),
    "efm_b200_decode_begin": (I32, [P, I32, I32, C.POINTER(I32), I32]),
    "efm_b200_set_token": (I32, [P, I32]),
    "efm_b200_decode_steps": (I32, [P, I32, I32]),
    "efm_b200_capture_decode": (I32, [P, I32]),
    "efm_b200_read_tokens": (I32, [P, C.POINTER(I32), I32, I32]),
    "efm_b200_read_logits": (I32, [P, C.POINTER(C.c_float), I32]),
    "efm_b200_synchronize": (I32, [P]),
    "efm_b200_event_record": (I32, [P, I32]),
    "efm_b200_event_elapsed_ms": (I32, [P, I32, I32, C.POINTER(C.c_float)]),
    "efm_b200_launch_count": (I32, [P, C.POINTER(C.c_int64)]),
    "efm_b200_decode_breakdown": (I32, [P, I32, C.POINTER(C.c_float)]),
    "efm_b200_decode_step_bytes": (I32, [P, I32, C.POINTER(C.c_int64)]),
    "efm_b200_op_gemv": (I32, [P, P, P, C.c_float, P, P, I32, I32]),
    "efm_b200_op_gemv_peer_consume": (I32, [P, P, P, C.c_float, P, I32, C.c_uint32, C.c_int64, P, P, I32, I32]),
    "efm_b200_op_gemm": (I32, [P, P, P, P, I32, I32, I32]),
    "efm_b200_op_decode_attention": (I32, [P, P, P, P, I32, I32, I32, I32, I32]),
    "efm_b200_op_decode_attention_noalloc": (I32, [P, P, P, P, I32, I32, I32, I32, I32]),
    "efm_b200_op_prefill_attention": (I32, [P, P, P, P, I32, I32, I32, I32, I32]),
    "efm_b200_op_sage_prefill_attention": (I32, [P, P, P, P, I32, I32, I32, I32, I32]),
    "efm_b200_set_prefill_attention": (I32, [P, I32]),
    "efm_b200_op_sample": (I32, [C.POINTER(C.c_float), I32, C.POINTER(Sampling), C.c_uint32, C.POINTER(I32)]),
    "efm_b200_op_segment_attention": (I32, [P, P, P, P, P, P, I32, I32, I32, I32]),
    "efm_b200_vit_create": (I32, [P, C.POINTER(VitDesc), C.POINTER(P)]),
    "efm_b200_vit_destroy": (I32, [P]),
    "efm_b200_vit_set_weight": (I32, [P, C.c_char_p, P, C.POINTER(C.c_int64), I32, I32, I32]),
    "efm_b200_vit_finalize_weights": (I32, [P]),
    "efm_b200_vit_plan": (I32, [C.POINTER(VitDesc), C.POINTER(I32), I32] + [C.POINTER(I32)] * 7),
    "efm_b200_vit_encode": (I32, [P, P, I32, C.POINTER(I32), I32, P, I32]),
    "efm_b200_vla_create": (I32, [C.POINTER(VlaDesc), I32, C.POINTER(P)]),
    "efm_b200_vla_destroy": (I32, [P]),
    "efm_b200_vla_last_error": (C.c_char_p, [P]),
    "efm_b200_vla_set_weight": (I32, [P, C.c_char_p, P, C.POINTER(C.c_int64), I32, I32, I32]),
    "efm_b200_vla_finalize_weights": (I32, [P]),
    "efm_b200_vla_chunk": (I32, [P, P, P, P, P, I32, P]),
    "efm_b200_vla_enqueue": (I32, [P]),
    "efm_b200_vla_stream": (I32, [P, C.POINTER(P)]),
    "efm_b200_vla_phase_ms": (I32, [P, C.POINTER(C.c_float)]),
    "efm_b200_vla_launch_count": (I32, [P, C.POINTER(C.c_int64), C.POINTER(C.c_int64)]),
}

_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: run `python edge-fm-x_b200/build.py` (there is no fallback path)")
        _lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(_lib, name)
            fn.restype, fn.argtypes = res, args
    return _lib


class BackendError(RuntimeError):
    pass


def _i32_array(values):
    return (I32 * len(values))(*[int(v) for v in values])


class Backend:
    """Thin object wrapper over one efm_b200_ctx."""

    def __init__(self, cfg, *, max_prefill_tokens=256, max_response_tokens=512, device_id=0, tp_rank=0, tp_size=1):
        self.L = lib()
        self.cfg = cfg
        d = ModelDesc()
        d.struct_size = C.sizeof(ModelDesc)
        d.num_layers, d.hidden, d.q_heads, d.kv_heads = cfg.num_layers, cfg.hidden, cfg.q_heads, cfg.kv_heads
        d.head_dim, d.intermediate, d.vocab = cfg.head_dim, cfg.intermediate, cfg.vocab
        d.rms_eps, d.rope_theta = cfg.rms_eps, cfg.rope_theta
        d.tied_lm_head = 1 if cfg.tied else 0
        d.use_mrope = 1 if cfg.mrope_section is not None else 0
        if cfg.mrope_section is not None:
            d.mrope_section[:] = cfg.mrope_section
        d.max_prefill_tokens, d.max_response_tokens = max_prefill_tokens, max_response_tokens
        self.ctx = P()
        st = self.L.efm_b200_create(C.byref(d), device_id, tp_rank, tp_size, C.byref(self.ctx))
        if st != EFM_OK:
            raise BackendError(f"create failed ({st}): {self.L.efm_b200_last_error(None).decode()}")

    def check(self, st, what=""):
        if st != EFM_OK:
            raise BackendError(f"{what} failed ({st}): {self.L.efm_b200_last_error(self.ctx).decode()}")

    def close(self):
        if self.ctx:
            self.L.efm_b200_destroy(self.ctx)
            self.ctx = P()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def tp_init(self, id_bytes):
        buf = C.create_string_buffer(bytes(id_bytes), 128)
        self.check(self.L.efm_b200_tp_init(self.ctx, buf), "tp_init")

    def tp_peer_export(self):
        buf = C.create_string_buffer(64)
        self.check(self.L.efm_b200_tp_peer_export(self.ctx, buf), "tp_peer_export")
        return bytes(buf.raw)

    def tp_peer_import(self, handles):
        """handles: list of the 64-byte exports of all ranks, in rank order."""
        blob = C.create_string_buffer(b"".join(handles), 64 * len(handles))
        self.check(self.L.efm_b200_tp_peer_import(self.ctx, blob, len(handles)), "tp_peer_import")

    def load_weights(self, weights):
        """weights: dict name -> torch bf16 tensor (CPU or CUDA)."""
        for name, t in weights.items():
            t = t.contiguous()
            shape = (C.c_int64 * t.dim())(*t.shape)
            mem = EFM_MEM_DEVICE if t.is_cuda else EFM_MEM_HOST
            if t.is_cuda:        # the backend copies on its own stream: the producer's work must be complete
                import torch
                torch.cuda.current_stream(t.device).synchronize()
            self.check(self.L.efm_b200_set_weight(self.ctx, name.encode(), P(t.data_ptr()), shape, t.dim(),
                                                  EFM_BF16, mem), "set_weight " + name)
        self.check(self.L.efm_b200_finalize_weights(self.ctx), "finalize_weights")

    def load_weights_partial(self, weights):
        """set_weight only (call finalize() after the last batch)."""
        for name, t in weights.items():
            t = t.contiguous()
            shape = (C.c_int64 * t.dim())(*t.shape)
            mem = EFM_MEM_DEVICE if t.is_cuda else EFM_MEM_HOST
            if t.is_cuda:
                import torch
                torch.cuda.current_stream(t.device).synchronize()
            self.check(self.L.efm_b200_set_weight(self.ctx, name.encode(), P(t.data_ptr()), shape, t.dim(),
                                                  EFM_BF16, mem), "set_weight " + name)

    def load_decode_weights_int4(self, tensors):
        """tensors: dict '<linear>.qweight' -> int8 tensor, '<linear>.scaling_factors' -> fp16 / bf16 tensor (before finalize)."""
        import torch
        codes = {torch.int8: 6, torch.uint8: 5, torch.float16: EFM_F16, torch.bfloat16: EFM_BF16}
        for name, t in tensors.items():
            t = t.contiguous()
            shape = (C.c_int64 * t.dim())(*t.shape)
            mem = EFM_MEM_DEVICE if t.is_cuda else EFM_MEM_HOST
            if t.is_cuda:
                torch.cuda.current_stream(t.device).synchronize()
            self.check(self.L.efm_b200_set_decode_weight(self.ctx, name.encode(), P(t.data_ptr()), shape, t.dim(), codes[t.dtype], mem),
                       "set_decode_weight " + name)

    def finalize(self):
        self.check(self.L.efm_b200_finalize_weights(self.ctx), "finalize_weights")

    def alloc_slot(self, slot, max_tokens):
        self.check(self.L.efm_b200_alloc_kv_slot(self.ctx, slot, max_tokens), "alloc_kv_slot")

    def set_sampling(self, temperature=0.0, top_p=1.0, seed=0, top_k=1):
        s = Sampling(temperature, top_p, top_k, 0, seed)
        self.check(self.L.efm_b200_set_sampling(self.ctx, C.byref(s)), "set_sampling")

    def prefill(self, slot, ids, kv_offset=0, embeds=None, embed_token_id=-1, pos3=None, sample=True):
        n = len(ids)
        ep, ne, em = None, 0, EFM_MEM_HOST
        if embeds is not None:
            embeds = embeds.contiguous()
            if embeds.is_cuda:
                import torch
                torch.cuda.current_stream(embeds.device).synchronize()
            ep, ne = P(embeds.data_ptr()), embeds.shape[0]
            em = EFM_MEM_DEVICE if embeds.is_cuda else EFM_MEM_HOST
        pp = None
        if pos3 is not None:
            flat = [int(v) for row in pos3 for v in row]
            assert len(flat) == 3 * n
            pp = _i32_array(flat)
        self.check(self.L.efm_b200_prefill(self.ctx, slot, _i32_array(ids), n, kv_offset, ep, ne, embed_token_id, em,
                                           pp, 1 if sample else 0), "prefill")

    def decode_begin(self, slot, kv_len, mrope_pos=None, step=1):
        mp = _i32_array(mrope_pos) if mrope_pos is not None else None
        self.check(self.L.efm_b200_decode_begin(self.ctx, slot, kv_len, mp, step), "decode_begin")

    def set_prefill_graph(self, enable):
        self.check(self.L.efm_b200_set_prefill_graph(self.ctx, 1 if enable else 0), "set_prefill_graph")

    def prefill_graph_stats(self):
        n, r = I32(), C.c_int64()
        self.check(self.L.efm_b200_prefill_graph_stats(self.ctx, C.byref(n), C.byref(r)), "prefill_graph_stats")
        return n.value, r.value

    def set_prefill_attention(self, kind):
        self.check(self.L.efm_b200_set_prefill_attention(self.ctx, int(kind)), "set_prefill_attention")

    def set_token(self, tok):
        self.check(self.L.efm_b200_set_token(self.ctx, int(tok)), "set_token")

    def decode_steps(self, n, use_graph=True):
        self.check(self.L.efm_b200_decode_steps(self.ctx, n, 1 if use_graph else 0), "decode_steps")

    def capture_decode(self, slot):
        self.check(self.L.efm_b200_capture_decode(self.ctx, slot), "capture_decode")

    def read_tokens(self, first, n):
        buf = (I32 * max(n, 1))()
        self.check(self.L.efm_b200_read_tokens(self.ctx, buf, first, n), "read_tokens")
        return list(buf[:n])

    def read_logits(self):
        import numpy as np
        out = np.empty(self.cfg.vocab, dtype=np.float32)
        self.check(self.L.efm_b200_read_logits(self.ctx, out.ctypes.data_as(C.POINTER(C.c_float)), self.cfg.vocab),
                   "read_logits")
        return out

    def synchronize(self):
        self.check(self.L.efm_b200_synchronize(self.ctx), "synchronize")

    def event_record(self, idx):
        self.check(self.L.efm_b200_event_record(self.ctx, idx), "event_record")

    def elapsed_ms(self, a, b):
        ms = C.c_float()
        self.check(self.L.efm_b200_event_elapsed_ms(self.ctx, a, b, C.byref(ms)), "event_elapsed")
        return ms.value

    def launch_count(self):
        n = C.c_int64()
        self.check(self.L.efm_b200_launch_count(self.ctx, C.byref(n)), "launch_count")
        return n.value

    def decode_breakdown(self, n_steps):
        out = (C.c_float * 7)()
        self.check(self.L.efm_b200_decode_breakdown(self.ctx, n_steps, out), "decode_breakdown")
        return dict(zip(("qkv", "attention", "o_proj", "gate_up", "down_proj", "lm_head", "sampler"), list(out)))

    def decode_step_bytes(self, kv_len):
        n = C.c_int64()
        self.check(self.L.efm_b200_decode_step_bytes(self.ctx, kv_len, C.byref(n)), "decode_step_bytes")
        return n.value

    def kv_layer(self, slot, layer):
        p, mt = P(), I32()
        self.check(self.L.efm_b200_kv_layer_ptr(self.ctx, slot, layer, C.byref(p), C.byref(mt)), "kv_layer_ptr")
        return p.value, mt.value


def vit_desc(vcfg, max_patches):
    d = VitDesc()
    d.struct_size = C.sizeof(VitDesc)
    d.depth, d.hidden, d.heads, d.intermediate = vcfg.depth, vcfg.hidden, vcfg.heads, vcfg.intermediate
    d.out_hidden, d.patch, d.temporal_patch, d.in_channels = vcfg.out_hidden, vcfg.patch, vcfg.temporal_patch, vcfg.in_channels
    d.merge, d.window, d.n_fullatt = vcfg.merge, vcfg.window, len(vcfg.fullatt)
    d.fullatt[:len(vcfg.fullatt)] = list(vcfg.fullatt)
    d.rms_eps, d.rope_theta, d.max_patches = vcfg.rms_eps, vcfg.rope_theta, max_patches
    return d


def vit_plan(vcfg, grids):
    """Host-only plan of the vision encoder (efm_b200_vit_plan) as python lists, or None when the grids are refused."""
    n = sum(t * h * w for t, h, w in grids)
    nm = n // (vcfg.merge * vcfg.merge)
    d = vit_desc(vcfg, max(n, vcfg.merge * vcfg.merge))
    bufs = [(I32 * max(nm, 1))()] + [(I32 * max(n, 1))() for _ in range(6)]
    st = lib().efm_b200_vit_plan(C.byref(d), _i32_array([v for g in grids for v in g]), len(grids), *bufs)
    if st != EFM_OK:
        return None
    names = ("order", "pos_h", "pos_w", "win_lo", "win_hi", "full_lo", "full_hi")
    return {k: list(b[:nm if k == "order" else n]) for k, b in zip(names, bufs)}


class VitEncoder:
    """Vision encoder bound to a Backend's device and stream (efm_b200_vit_*)."""

    def __init__(self, be: Backend, vcfg, max_patches):
        self.be, self.L, self.cfg = be, be.L, vcfg
        d = vit_desc(vcfg, max_patches)
        self.h = P()
        be.check(self.L.efm_b200_vit_create(be.ctx, C.byref(d), C.byref(self.h)), "vit_create")

    def close(self):
        if self.h:
            self.L.efm_b200_vit_destroy(self.h)
            self.h = P()

    def load_weights(self, weights):
        for name, t in weights.items():
            t = t.contiguous()
            shape = (C.c_int64 * t.dim())(*t.shape)
            if t.is_cuda:
                import torch
                torch.cuda.current_stream(t.device).synchronize()
            self.be.check(self.L.efm_b200_vit_set_weight(self.h, name.encode(), P(t.data_ptr()), shape, t.dim(), EFM_BF16,
                                                         EFM_MEM_DEVICE if t.is_cuda else EFM_MEM_HOST), "vit_set_weight " + name)
        self.be.check(self.L.efm_b200_vit_finalize_weights(self.h), "vit_finalize_weights")

    def encode(self, pixels, grids, out):
        """pixels, out: torch bf16 tensors (CPU or CUDA); grids: list of (t, h, w)."""
        pixels = pixels.contiguous()
        if pixels.is_cuda or out.is_cuda:
            import torch
            torch.cuda.current_stream().synchronize()
        flat = _i32_array([v for g in grids for v in g])
        self.be.check(self.L.efm_b200_vit_encode(self.h, P(pixels.data_ptr()), EFM_MEM_DEVICE if pixels.is_cuda else EFM_MEM_HOST,
                                                 flat, len(grids), P(out.data_ptr()),
                                                 EFM_MEM_DEVICE if out.is_cuda else EFM_MEM_HOST), "vit_encode")
        return out


def vla_desc(cfg):
    """efm_vla_desc from an oracle.smolvla.VlaConfig-like object."""
    d = VlaDesc()
    d.struct_size = C.sizeof(VlaDesc)
    for name, _ in VlaDesc._fields_[1:]:
        setattr(d, name, getattr(cfg, name))
    return d


class VlaPolicy:
    """Action-chunk model behind efm_b200_vla_* (owns its device buffers and stream)."""

    def __init__(self, cfg, device=0):
        self.L, self.cfg = lib(), cfg
        d = vla_desc(cfg)
        self.h = P()
        st = self.L.efm_b200_vla_create(C.byref(d), device, C.byref(self.h))
        if st != 0:
            raise RuntimeError(f"vla_create failed with status {st}")

    def check(self, st, what):
        if st != 0:
            raise RuntimeError(f"{what}: status {st}: {self.L.efm_b200_vla_last_error(self.h).decode()}")

    def close(self):
        if self.h:
            self.L.efm_b200_vla_destroy(self.h)
            self.h = P()

    def load_weights(self, weights):
        for name, t in weights.items():
            t = t.contiguous()
            shape = (C.c_int64 * t.dim())(*t.shape)
            self.check(self.L.efm_b200_vla_set_weight(self.h, name.encode(), P(t.data_ptr()), shape, t.dim(), EFM_BF16,
                                                      EFM_MEM_DEVICE if t.is_cuda else EFM_MEM_HOST), "vla_set_weight " + name)
        self.check(self.L.efm_b200_vla_finalize_weights(self.h), "vla_finalize_weights")

    def chunk(self, images, ids, state, noise):
        """Host tensors in (fp32 / int32), host fp32 [chunk, action_dim] out."""
        import torch
        c = self.cfg
        images, state, noise = (t.to(torch.float32).contiguous() for t in (images, state, noise))
        ids = ids.to(torch.int32).contiguous()
        out = torch.empty(c.chunk, c.action_dim, dtype=torch.float32)
        self.check(self.L.efm_b200_vla_chunk(self.h, P(images.data_ptr()), P(ids.data_ptr()), P(state.data_ptr()),
                                             P(noise.data_ptr()), EFM_MEM_HOST, P(out.data_ptr())), "vla_chunk")
        return out

    def enqueue(self):
        self.check(self.L.efm_b200_vla_enqueue(self.h), "vla_enqueue")

    def stream(self):
        s = P()
        self.check(self.L.efm_b200_vla_stream(self.h, C.byref(s)), "vla_stream")
        return s.value

    def phase_ms(self):
        ms = (C.c_float * 4)()
        self.check(self.L.efm_b200_vla_phase_ms(self.h, ms), "vla_phase_ms")
        return dict(zip(("vision", "prefix", "bridge", "denoise"), [float(x) for x in ms]))

    def launch_count(self):
        a, b = C.c_int64(), C.c_int64()
        self.check(self.L.efm_b200_vla_launch_count(self.h, C.byref(a), C.byref(b)), "vla_launch_count")
        return a.value, b.value


def generate(be: Backend, slot, prompt, max_new_tokens, *, prefix_len=0, embeds=None, embed_token_id=-1, pos3=None,
             mrope_last_pos=None, use_graph=True, forced=None, collect_logits=False):
    """generate() through the C ABI: prefill of prompt[prefix_len:], then decode steps.
    forced: teacher-forced feed tokens (step by step, no graph batching).  Returns (tokens, logits list)."""
    ids = list(prompt[prefix_len:])
    p3 = None if pos3 is None else [list(r[prefix_len:]) for r in pos3]
    be.prefill(slot, ids, kv_offset=prefix_len, embeds=embeds, embed_token_id=embed_token_id, pos3=p3, sample=True)
    logits = [be.read_logits()] if collect_logits else []
    mp = None
    if be.cfg.mrope_section is not None:
        if mrope_last_pos is None:
            mrope_last_pos = [max(max(r) for r in pos3)] * 3
        mp = [m + 1 for m in mrope_last_pos]
    n_dec = max_new_tokens - 1
    if n_dec > 0:
        be.decode_begin(slot, len(prompt), mp, 1)
        if forced is None and not collect_logits:
            be.decode_steps(n_dec, use_graph)
        else:
            for s in range(n_dec):
                if forced is not None:
                    be.set_token(forced[s])
                be.decode_steps(1, use_graph)
                if collect_logits:
                    logits.append(be.read_logits())
    return be.read_tokens(0, max_new_tokens), logits


def tp_unique_id():
    buf = C.create_string_buffer(128)
    st = lib().efm_b200_tp_unique_id(buf)
    if st != EFM_OK:
        raise BackendError(f"tp_unique_id failed ({st}): {lib().efm_b200_last_error(None).decode()}")
    return bytes(buf.raw)
