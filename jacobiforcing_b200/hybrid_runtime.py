"""HybridRuntime — Python host of libjf_hybrid.so: the per-rank pieces a model runner owns for a layered hybrid decoder
(weights by checkpoint name, the paged key cache, recurrent-state slots) and the step function over a packed batch of
entries.  numpy carries host buffers across the ABI; torch is not needed."""
from __future__ import annotations

import ctypes as C
import glob
import os
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from . import _hybrid_cabi as cabi
from .hybrid_config import HybridConfig, iter_safetensors

DTYPES = {"bfloat16": 0, "float32": 1}


def _i32(x) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(x, dtype=np.int32))


def _ptr(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


class HybridRuntime:
    def __init__(self, config: HybridConfig, *, dtype: str = "bfloat16", device: int = 0, max_step_tokens: int = 2048,
                 max_step_entries: int = 64, page_size: int = 256, num_pages: int = 64, max_pages_per_seq: int = 64,
                 num_slots: int = 8, max_want: int = 0):
        if dtype not in DTYPES:
            raise ValueError(f"dtype must be one of {sorted(DTYPES)}")
        self.lib = cabi.load()
        self.config = config
        self.dtype = dtype
        self.vocab, self.width = config.vocab, config.width
        self.page_size, self.num_pages, self.num_slots = page_size, num_pages, num_slots
        self.max_step_tokens, self.max_step_entries = max_step_tokens, max_step_entries
        self.max_pages_per_seq = max_pages_per_seq
        self.max_want = max_want or max_step_tokens
        m = cabi.ModelCfg(config.width, config.vocab, len(config.layers), DTYPES[dtype], config.emb_scale,
                          config.logit_scale, config.norm_eps, config.norm_kind, config.block_kind, config.pos_kind,
                          int(config.embed_norm), int(config.tied_head), config.resid_mult, config.canon_taps,
                          config.side_dim, config.depth_avg, config.pair_buckets, config.pair_mul_prev, config.pair_mul_cur)
        layers = (cabi.LayerCfg * len(config.layers))()
        for i, s in enumerate(config.layers):
            for name, _ in cabi.LayerCfg._fields_:
                setattr(layers[i], name, getattr(s, name))
        rt = cabi.RuntimeCfg(device, max_step_tokens, max_step_entries, page_size, num_pages, max_pages_per_seq, num_slots,
                             self.max_want)
        h = C.c_void_p()
        cabi.check(self.lib.hy_create(C.byref(m), layers, C.byref(rt), C.byref(h)), None)
        self.h = h
        self.stats = {"steps": 0, "tokens": 0, "device_ms": 0.0}

    # ---- lifecycle -------------------------------------------------------------------------------------------------
    def close(self):
        if getattr(self, "h", None):
            self.lib.hy_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- weights ---------------------------------------------------------------------------------------------------
    def load_tensor(self, name: str, dtype_code: int, shape: Sequence[int], data: np.ndarray) -> None:
        shp = (C.c_int64 * max(1, len(shape)))(*shape)
        cabi.check(self.lib.hy_load_tensor(self.h, name.encode(), data.ctypes.data_as(C.c_void_p), shp, len(shape),
                                           dtype_code), self.h)

    def load_dir(self, path: str) -> None:
        files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
        if not files:
            raise FileNotFoundError(f"no *.safetensors under {path}")
        for f in files:
            for name, code, shape, data in iter_safetensors(f):
                self.load_tensor(name, code, shape, data)
        self.finalize()

    def load_state_dict(self, sd: Dict[str, "object"]) -> None:
        """Tensors by checkpoint name: numpy float32 / int32 arrays, or torch tensors (bfloat16 / float32 / int32)."""
        for name, t in sd.items():
            if hasattr(t, "detach"):                                   # torch tensor, without importing torch here
                t = t.detach().cpu().contiguous()
                kind = str(t.dtype)
                if kind == "torch.bfloat16":
                    import torch
                    a = t.view(torch.int16).numpy().view(np.uint16)
                    self.load_tensor(name, 0, list(t.shape), np.ascontiguousarray(a))
                    continue
                t = t.float().numpy() if kind != "torch.int32" else t.numpy()
            a = np.ascontiguousarray(t)
            if a.dtype == np.float32:
                self.load_tensor(name, 1, list(a.shape), a)
            elif a.dtype == np.int32:
                self.load_tensor(name, 3, list(a.shape), a)
            else:
                self.load_tensor(name, 1, list(a.shape), np.ascontiguousarray(a.astype(np.float32)))
        self.finalize()

    def finalize(self) -> None:
        cabi.check(self.lib.hy_finalize(self.h), self.h)

    # ---- one step ---------------------------------------------------------------------------------------------------
    def step(self, entries: Sequence[Tuple[Sequence[int], int, int, Sequence[int]]], want: Sequence[int] = (),
             *, want_logits: bool = True, sample: bool = False, temperature: Optional[Sequence[float]] = None,
             seed: int = 0, want_layers: bool = False):
        """entries: (tokens, pos0, slot, pages) per request; want: indices into the packed token list.
        Returns {"logits": [n_want, vocab] float32 or None, "sampled": int32 [n_want] or None, "layers": ...}."""
        E = len(entries)
        toks: List[int] = []
        start = [0]
        pages = np.zeros((E, self.max_pages_per_seq), dtype=np.int32)
        for e, (t, pos0, slot, pg) in enumerate(entries):
            toks.extend(int(x) for x in t)
            start.append(len(toks))
            if len(pg) > self.max_pages_per_seq:
                raise RuntimeError("request holds more pages than max_pages_per_seq")
            pages[e, :len(pg)] = pg
        T = len(toks)
        n_want = len(want)
        logits = np.empty((n_want, self.vocab), dtype=np.float32) if (n_want and want_logits) else None
        sampled = np.empty((n_want,), dtype=np.int32) if (n_want and sample) else None
        temp = np.ascontiguousarray(np.asarray(temperature, dtype=np.float32)) if (temperature is not None and n_want) else None
        layers = np.empty((len(self.config.layers), T, self.width), dtype=np.float32) if want_layers else None
        a_tok, a_start = _i32(toks), _i32(start)
        a_pos0, a_slot = _i32([e[1] for e in entries]), _i32([e[2] for e in entries])
        a_want = _i32(list(want)) if n_want else None
        cabi.check(self.lib.hy_step(self.h, E, _ptr(a_tok), _ptr(a_start), _ptr(a_pos0), _ptr(a_slot), _ptr(pages), n_want,
                                    _ptr(a_want), _ptr(logits), _ptr(sampled), _ptr(temp), C.c_uint64(seed & (2 ** 64 - 1)),
                                    _ptr(layers)), self.h)
        self.stats["steps"] += 1
        self.stats["tokens"] += T
        self.stats["device_ms"] += float(self.lib.hy_last_step_ms(self.h))
        return {"logits": logits, "sampled": sampled, "layers": layers}

    def profile(self, on: bool) -> None:
        cabi.check(self.lib.hy_profile_enable(self.h, 1 if on else 0), self.h)

    def profile_read(self) -> Dict[str, float]:
        ms = (C.c_float * len(cabi.PROFILE_CATEGORIES))()
        cabi.check(self.lib.hy_profile_read(self.h, ms), self.h)
        return dict(zip(cabi.PROFILE_CATEGORIES, (float(x) for x in ms)))

    @property
    def launches(self) -> int:
        return int(self.lib.hy_launch_count(self.h))

    def memory_info(self) -> Dict[str, int]:
        v = [C.c_int64() for _ in range(4)]
        cabi.check(self.lib.hy_memory_info(self.h, *[C.byref(x) for x in v]), self.h)
        return dict(zip(("weights", "cache", "state", "workspace"), (int(x.value) for x in v)))
