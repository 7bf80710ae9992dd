"""Host-side mirror of one serving stage (a contiguous layer range resident on one GPU).

Mirrors what a mesh-llm worker is to its caller: it is created for blk.[layer_begin, layer_end),
loads its own tensors by GGUF name, and runs micro-batches, handing the [rows x n_embd] f32
activation to the next stage.  All compute happens in libb200kq.so.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import capi
from .capi import StageConfig, check, lib, ptr, cur_stream

_DEFAULTS = dict(n_expert=0, n_expert_used=0, n_ff_exp=0, n_ff=0, n_seq=1, rope_neox=1, qkv_bias=0,
                 qk_norm=0, has_embd=1, has_output=1, rms_eps=1e-6, rope_theta=1e6, layer_begin=0,
                 n_ubatch=512, device=0, n_vocab=0)


class Stage:
    def __init__(self, **kw):
        cfg = dict(_DEFAULTS)
        cfg.update(kw)
        cfg.setdefault("layer_end", cfg["n_layer"])
        self.cfg = StageConfig(**cfg)
        self.device = torch.device("cuda", self.cfg.device)
        h = C.c_void_p()
        check(lib().b200_stage_create(C.byref(self.cfg), C.byref(h)))
        self.h = h

    @classmethod
    def from_gguf(cls, gguf_file, layer_begin=0, layer_end=-1, n_ctx=4096, n_seq=1, n_ubatch=512, device=0):
        """Stage for blk.[layer_begin, layer_end) of the model in `gguf_file` (a GgufFile), with exactly
        its own tensors read from the file.  Returns (stage, tensors loaded, bytes read)."""
        cfg = gguf_file.stage_config(layer_begin, layer_end, n_ctx, n_seq, n_ubatch, device)
        st = cls(**{name: getattr(cfg, name) for name, _ in StageConfig._fields_})
        n, nbytes = C.c_int64(), C.c_int64()
        check(lib().b200_stage_load_gguf(st.h, gguf_file.h, C.byref(n), C.byref(nbytes)))
        return st, n.value, nbytes.value

    def tensor_names(self):
        out = []
        for i in range(lib().b200_stage_tensor_count(self.h)):
            name = C.create_string_buffer(128)
            ty, ne = C.c_uint32(), (C.c_int64 * 3)()
            check(lib().b200_stage_tensor_info(self.h, i, name, 128, C.byref(ty), C.byref(ne)))
            out.append((name.value.decode(), ty.value, list(ne)))
        return out

    def close(self):
        if getattr(self, "h", None):
            lib().b200_stage_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- weights ------------------------------------------------------------------------------
    def set_tensor(self, name, type_, data):
        data = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        check(lib().b200_stage_set_tensor(self.h, name.encode(), type_, data.ctypes.data, data.size))

    def get_tensor(self, name, nbytes):
        out = np.empty(nbytes, np.uint8)
        check(lib().b200_stage_get_tensor(self.h, name.encode(), out.ctypes.data, nbytes))
        return out

    def load(self, tensors):
        """tensors: iterable of (name, ggml_type, bytes-like) in GGUF layout"""
        for name, type_, data in tensors:
            self.set_tensor(name, type_, data)

    def generate(self, seed):
        check(lib().b200_stage_generate(self.h, seed))

    def weight_bytes(self):
        return lib().b200_stage_weight_bytes(self.h)

    def kernel_launches(self):
        return lib().b200_stage_kernel_launches(self.h)

    # ---- compute ------------------------------------------------------------------------------
    def forward(self, tokens=None, hidden_in=None, n_seq=1, T=None, pos0=0, hidden_out=None,
                logits=None, all_logits=False, next_tokens=None, seq0=0):
        """Device tensors in, device tensors out (allocated when not supplied).
        rows are sequence-major: row = seq * T + t."""
        c = self.cfg
        if tokens is not None:
            rows = tokens.numel()
        else:
            rows = hidden_in.shape[0]
        T = rows // n_seq if T is None else T
        if hidden_out is None and not c.has_output:
            hidden_out = torch.empty((rows, c.n_embd), dtype=torch.float32, device=self.device)
        if c.has_output:
            if logits is None:
                logits = torch.empty((rows if all_logits else n_seq, c.n_vocab), dtype=torch.float32,
                                     device=self.device)
            if next_tokens is None:
                next_tokens = torch.empty(rows if all_logits else n_seq, dtype=torch.int32,
                                          device=self.device)
        check(lib().b200_stage_forward(self.h, ptr(tokens), ptr(hidden_in), seq0, n_seq, T, pos0,
                                       ptr(hidden_out), ptr(logits), int(all_logits),
                                       ptr(next_tokens), cur_stream()))
        return hidden_out, logits, next_tokens

    def set_expert_mask(self, mask):
        """mask: one entry per expert (nonzero = allowed) or None to clear it; as the reference's
        llama_model_set_expert_mask, a mask of the wrong length is refused"""
        if mask is None:
            check(lib().b200_stage_set_expert_mask(self.h, None, 0))
            return
        m = np.ascontiguousarray(np.asarray(mask) != 0, dtype=np.uint8)
        check(lib().b200_stage_set_expert_mask(self.h, m.ctypes.data, m.size))

    def peek(self, which, shape):
        """diagnostics: an internal activation buffer ("q", "k", "v", "att", "g", "x") after the last forward"""
        out = np.empty(shape, np.float32)
        check(lib().b200_stage_peek(self.h, which.encode(), out.ctypes.data, out.size))
        return out

    def synchronize(self):
        check(lib().b200_stage_synchronize(self.h))
