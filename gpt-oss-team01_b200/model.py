"""Whole-model greedy decode over the C ABI (``gptoss_model_*``): the lock-step batched loop of the
reference's ``inference`` (getp-csrc/submit/getp_run_submit.cpp:60-96) on one GPU."""
from __future__ import annotations

import ctypes as C
import dataclasses

import numpy as np

from . import binfmt, capi
from .moe import GptossError

EOS_IDS = (199999, 200002)  # run.cpp:939, getp_run_submit.cpp:249


class Model:
    def __init__(self, cfg: binfmt.Config, device=0, max_batch=1, max_seq=None):
        self.lib = capi.load()
        self.cfg = cfg
        self.max_batch = max_batch
        self.max_seq = max_seq or cfg.seq_len
        self._m = C.c_void_p()
        c = capi.ModelConfig(*dataclasses.astuple(cfg))
        rc = self.lib.gptoss_model_create(C.byref(c), device, max_batch, self.max_seq, C.byref(self._m))
        if rc != capi.OK:
            self._m = C.c_void_p()
            raise GptossError(rc, "gptoss_model_create failed (unsupported dimensions, no sm_100 device, or out of memory)")

    def _check(self, rc):
        if rc != capi.OK:
            raise GptossError(rc, self.lib.gptoss_model_last_error(self._m).decode())

    def close(self):
        if self._m:
            self.lib.gptoss_model_destroy(self._m)
            self._m = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def load_bin(self, path):
        self._check(self.lib.gptoss_model_load_bin(self._m, str(path).encode()))

    def fill_synthetic(self, seed, sigma=0.02):
        self._check(self.lib.gptoss_model_fill_synthetic(self._m, seed, sigma))

    def step(self, tokens, pos, need_next=True):
        """tokens: int32 [B] -> greedy next tokens int32 [B] (None with need_next=False: the classifier is skipped)"""
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        nxt = np.empty_like(tokens) if need_next else None
        self._check(self.lib.gptoss_model_step(self._m, tokens.ctypes.data_as(C.c_void_p), int(pos), tokens.size,
                                               nxt.ctypes.data_as(C.c_void_p) if need_next else None))
        return nxt

    def logits(self, row=0):
        out = np.empty(self.cfg.vocab_size, np.float32)
        self._check(self.lib.gptoss_model_read_logits(self._m, row, out.ctypes.data_as(C.c_void_p)))
        return out

    def generate(self, prompts, n_generate, stop_on_eos=False):
        """prompts: int32 [B, n_prompt] (same length).  Returns int32 [B, n_generate]: the greedy continuation,
        prompt tokens force-fed one position per step; a sequence that emits an end-of-sequence id keeps
        running in lock-step (its later tokens are ignored by the caller) unless stop_on_eos trims them to -1."""
        prompts = np.ascontiguousarray(prompts, dtype=np.int32)
        B, n_prompt = prompts.shape
        out = np.full((B, n_generate), -1, np.int32)
        done = np.zeros(B, bool)
        tok = prompts[:, 0].copy()
        for pos in range(n_prompt + n_generate - 1):
            nxt = self.step(tok, pos, need_next=pos + 1 >= n_prompt)
            if pos + 1 < n_prompt:
                tok = prompts[:, pos + 1].copy()
            else:
                g = pos + 1 - n_prompt
                out[:, g] = np.where(done, -1, nxt) if stop_on_eos else nxt
                if stop_on_eos:
                    done |= np.isin(nxt, EOS_IDS)
                tok = nxt
        return out
