"""Whole-model greedy decode over the C ABI (``gptoss_model_*``): the lock-step batched loop of the
reference's ``inference`` (getp-csrc/submit/getp_run_submit.cpp:60-96) on one GPU, or as one rank of a group of
GPUs that decode a batch together (sequences dealt out in slices, experts sharded; getp-csrc/src/model.cpp:153-489)."""
from __future__ import annotations

import ctypes as C
import dataclasses

import numpy as np

from . import binfmt, capi
from .moe import GptossError

EOS_IDS = (199999, 200002)  # run.cpp:939, getp_run_submit.cpp:249


class Model:
    def __init__(self, cfg: binfmt.Config, device=0, max_batch=1, max_seq=None, rank=0, world=1):
        """max_batch: batch of the whole group; a rank of a group holds its slice of the sequences (``slice``)."""
        self.lib = capi.load()
        self.cfg = cfg
        self.max_batch = max_batch
        self.max_seq = max_seq or cfg.seq_len
        self.rank, self.world = rank, world
        self._m = C.c_void_p()
        c = capi.ModelConfig(*dataclasses.astuple(cfg))
        rc = self.lib.gptoss_model_create_ep(C.byref(c), device, rank, world, max_batch, self.max_seq, C.byref(self._m))
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

    # ---- groups of GPUs -------------------------------------------------------------------------------------
    def slice(self, batch):
        """(first sequence, number of sequences) of this rank for a batch of ``batch`` sequences of the group."""
        first, count = C.c_int(), C.c_int()
        self._check(self.lib.gptoss_model_slice(self._m, int(batch), C.byref(first), C.byref(count)))
        return first.value, count.value

    def _ctx(self):
        return C.c_void_p(self.lib.gptoss_model_moe_ctx(self._m))

    def comm_export(self) -> bytes:
        """This rank's CUDA IPC handle; exchange the handles of all ranks (rank order) and pass them to comm_attach."""
        buf = C.create_string_buffer(capi.IPC_HANDLE_BYTES)
        self._check(self.lib.gptoss_comm_export(self._ctx(), buf))
        return buf.raw

    def comm_attach(self, handles):
        blob = b"".join(handles)
        assert len(blob) == self.world * capi.IPC_HANDLE_BYTES
        self._check(self.lib.gptoss_comm_attach(self._ctx(), blob))

    def attach_peers(self, group=None):
        """One process per GPU: exchanges the IPC handles over torch.distributed and attaches all ranks."""
        import torch.distributed as dist
        gathered = [None] * self.world
        dist.all_gather_object(gathered, self.comm_export(), group=group)
        self.comm_attach(gathered)
        dist.barrier(group=group)

    @staticmethod
    def attach_local(models):
        """Attaches the ranks of a group whose model objects live in this process (rank order)."""
        arr = (C.c_void_p * len(models))(*[m._ctx() for m in models])
        for m in models:
            m._check(m.lib.gptoss_comm_attach_local(m._ctx(), arr))

    def set_peer_timeout_ms(self, ms):
        self._check(self.lib.gptoss_comm_set_timeout_ms(self._ctx(), int(ms)))

    # ---- steps ----------------------------------------------------------------------------------------------
    def step(self, tokens, pos, need_next=True, batch=None):
        """tokens: int32 ids of this rank's sequences -> their greedy next tokens (None with need_next=False: the
        classifier is skipped).  ``batch``: batch of the whole group (default: len(tokens), the single-GPU case)."""
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        nxt = np.empty_like(tokens) if need_next else None
        self._check(self.lib.gptoss_model_step(self._m, tokens.ctypes.data_as(C.c_void_p), int(pos),
                                               tokens.size if batch is None else int(batch),
                                               nxt.ctypes.data_as(C.c_void_p) if need_next else None))
        return nxt

    def step_rows(self, tokens, rows, pos, need_next=True):
        """A step of a compacted batch: ``tokens[i]`` is the input of the live sequence whose KV-cache row is ``rows[i]``."""
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        rows = np.ascontiguousarray(rows, dtype=np.int32)
        assert tokens.shape == rows.shape
        nxt = np.empty_like(tokens) if need_next else None
        self._check(self.lib.gptoss_model_step_rows(self._m, tokens.ctypes.data_as(C.c_void_p), rows.ctypes.data_as(C.c_void_p),
                                                    int(pos), tokens.size, nxt.ctypes.data_as(C.c_void_p) if need_next else None))
        return nxt

    def step_seqs(self, tokens, rows, positions, need_next=True):
        """A step of sequences that did not start together (continuous batching): sequence i takes ``tokens[i]`` at
        position ``positions[i]`` and lives in KV-cache row ``rows[i]``."""
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        rows = np.ascontiguousarray(rows, dtype=np.int32)
        positions = np.ascontiguousarray(positions, dtype=np.int32)
        assert tokens.shape == rows.shape == positions.shape
        nxt = np.empty_like(tokens) if need_next else None
        self._check(self.lib.gptoss_model_step_seqs(self._m, tokens.ctypes.data_as(C.c_void_p), rows.ctypes.data_as(C.c_void_p),
                                                    positions.ctypes.data_as(C.c_void_p), tokens.size,
                                                    nxt.ctypes.data_as(C.c_void_p) if need_next else None))
        return nxt

    @staticmethod
    def step_group(models, tokens, pos, need_next=True):
        """One step of a whole group driven from this thread: ``tokens`` int32 [B] for the whole batch; every phase
        runs for every rank before the next phase starts (a rank's device-side waits are then already satisfied)."""
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        B = tokens.size
        parts = []
        for m in models:
            first, n = m.slice(B)
            part = np.ascontiguousarray(tokens[first:first + n])
            parts.append((first, n, part))
            m._check(m.lib.gptoss_model_step_begin(m._m, part.ctypes.data_as(C.c_void_p), int(pos), B))
        for layer in range(models[0].cfg.n_layers):
            for m in models:
                m._check(m.lib.gptoss_model_layer_attention(m._m, layer))
            for m in models:
                m._check(m.lib.gptoss_model_layer_moe_dispatch(m._m, layer))
            for m in models:
                m._check(m.lib.gptoss_model_layer_moe_push(m._m, layer))
            for m in models:
                m._check(m.lib.gptoss_model_layer_moe_combine(m._m, layer))
        nxt = np.empty(B, np.int32) if need_next else None
        for m, (first, n, _) in zip(models, parts):
            out = np.empty(n, np.int32)
            m._check(m.lib.gptoss_model_step_end(m._m, out.ctypes.data_as(C.c_void_p) if need_next else None))
            if need_next:
                nxt[first:first + n] = out
        return nxt

    def logits(self, row=0):
        out = np.empty(self.cfg.vocab_size, np.float32)
        self._check(self.lib.gptoss_model_read_logits(self._m, row, out.ctypes.data_as(C.c_void_p)))
        return out

    def generate(self, prompts, n_generate, stop_on_eos=False, batch=None, first_pos=0):
        """prompts: int32 [B, n_prompt] (same length).  Returns int32 [B, n_generate]: the greedy continuation,
        prompt tokens force-fed one position per step; a sequence that emits an end-of-sequence id keeps
        running in lock-step (its later tokens are ignored by the caller) unless stop_on_eos trims them to -1.
        In a group, ``prompts`` holds this rank's sequences and ``batch`` is the batch of the whole group; every
        rank must call generate with the same prompt length and n_generate.  ``first_pos`` shifts the positions (the
        cache rows before it keep whatever they held: for timing a step at a long context without decoding up to it)."""
        prompts = np.ascontiguousarray(prompts, dtype=np.int32)
        B, n_prompt = prompts.shape
        out = np.full((B, n_generate), -1, np.int32)
        done = np.zeros(B, bool)
        tok = prompts[:, 0].copy()
        for pos in range(n_prompt + n_generate - 1):
            nxt = self.step(tok, first_pos + pos, need_next=pos + 1 >= n_prompt, batch=batch)
            if pos + 1 < n_prompt:
                tok = prompts[:, pos + 1].copy()
            else:
                g = pos + 1 - n_prompt
                out[:, g] = np.where(done, -1, nxt) if stop_on_eos else nxt
                if stop_on_eos:
                    done |= np.isin(nxt, EOS_IDS)
                tok = nxt
        return out
