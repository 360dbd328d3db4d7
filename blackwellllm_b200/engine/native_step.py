"""The decode step's hot path behind one C call (``csrc/decode_step.cu``, declared in
``csrc/decode_step.h``): reconcile positions, reserve pages, pack, copy to the device, replay
the captured graph, choose the tokens greedily, read them back.  Python hands over the
buffers it owns and gets a status code; on anything but success it takes its ordinary path,
which raises the error with its explanation.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import numpy as np
import torch

from ..cache.manager import native as host_runtime
from ..kernels.build import load_library

SUCCESS = 0
STATUS_NAMES = {0: "Success", 1: "CudaRuntimeError", 2: "OutOfPages", 3: "InvalidArgument", 4: "InvalidConfig",
                5: "StateMismatch"}


class DecodeStepArgs(ctypes.Structure):
    _fields_ = [("cache", ctypes.c_void_p), ("n", ctypes.c_int), ("handles", ctypes.c_void_p),
                ("tokens", ctypes.c_void_p), ("positions", ctypes.c_void_p), ("device_tokens", ctypes.c_void_p),
                ("vocab", ctypes.c_int), ("table_width", ctypes.c_int), ("max_context", ctypes.c_longlong),
                ("pinned", ctypes.c_void_p), ("pinned_words", ctypes.c_longlong), ("device_step", ctypes.c_void_p),
                ("step_words", ctypes.c_longlong), ("graph_exec", ctypes.c_void_p), ("stream", ctypes.c_void_p),
                ("logits", ctypes.c_void_p), ("logits_ld", ctypes.c_longlong), ("sampled_device", ctypes.c_void_p),
                ("sampled_host", ctypes.c_void_p), ("wait", ctypes.c_int), ("cuda_error", ctypes.c_int)]


_lib = None


def library():
    """The decode-step library, bound once to the host runtime's and the sampler's entry points."""
    global _lib
    if _lib is None:
        lib = load_library("decode_step")
        lib.bw_decode_step.argtypes = [ctypes.POINTER(DecodeStepArgs)]
        lib.bw_decode_step.restype = ctypes.c_int
        lib.bw_decode_step_bind.argtypes = [ctypes.c_void_p] * 4
        lib.bw_decode_step_bind.restype = ctypes.c_int
        rt, sampling = host_runtime(), load_library("sampling")

        def addr(fn):
            return ctypes.cast(fn, ctypes.c_void_p).value
        if lib.bw_decode_step_bind(addr(rt.bwh_pack_step), addr(rt.bwh_length), addr(rt.bwh_truncate),
                                   addr(sampling.bw_sample)) != SUCCESS:
            raise RuntimeError("bw_decode_step_bind refused its entry points")
        _lib = lib
    return _lib


class NativeDecodeSlot:
    """What one batch size's native step keeps between calls: the argument block and the small arrays it
    points at (handles, tokens, positions), the sampled tokens on the device."""

    def __init__(self, engine, n: int, graph_slot: dict):
        self.n = n
        self.handles = np.zeros(n, dtype=np.int32)
        self.tokens = np.zeros(n, dtype=np.int32)
        self.positions = np.zeros(n, dtype=np.int32)
        self.sampled = torch.empty(n, dtype=torch.int32, device=engine.device)
        # where the sampled tokens land on the host: a small ring, so that a caller who queues the next
        # step before reading this one's tokens (up to three steps ahead) still finds them
        self.host_ring = [torch.empty(n, dtype=torch.int32, pin_memory=True) for _ in range(4)]
        self.turn = 0
        logits = graph_slot["logits"]
        a = DecodeStepArgs()
        a.cache, a.n = engine.cache._h, n
        a.handles, a.tokens, a.positions = self.handles.ctypes.data, self.tokens.ctypes.data, self.positions.ctypes.data
        a.vocab, a.table_width = engine.config.vocab_size, engine._graph_width
        a.max_context = engine.options.max_context or (1 << 40)
        a.device_step, a.step_words = graph_slot["buf"].data_ptr(), graph_slot["buf"].numel()
        a.graph_exec = graph_slot["graph"].raw_cuda_graph_exec()
        a.logits, a.logits_ld = logits.data_ptr(), logits.stride(0)
        a.sampled_device = self.sampled.data_ptr()
        self.args = a


def decode_step(engine, slot: NativeDecodeSlot, rids, tokens, positions, token_source: Optional[torch.Tensor],
                wait: bool):
    """Runs the step; returns (status, pinned host tensor of the sampled tokens or None)."""
    cache = engine.cache
    n = slot.n
    for i, rid in enumerate(rids):
        h = cache.handle(rid)
        if h < 0:
            return 5, None                      # a sequence the cache does not hold yet: the ordinary path creates it
        slot.handles[i] = h
    slot.tokens[:] = tokens
    slot.positions[:] = positions
    a = slot.args
    pinned = engine._builder.pinned(int(a.step_words))
    ring = engine._builder.last_ring_slot
    host = slot.host_ring[slot.turn]
    slot.turn = (slot.turn + 1) % len(slot.host_ring)
    a.pinned, a.pinned_words = pinned.data_ptr(), pinned.numel()
    a.device_tokens = token_source.data_ptr() if token_source is not None else None
    a.stream = torch.cuda.current_stream(engine.device).cuda_stream
    a.sampled_host, a.wait = host.data_ptr(), int(wait)
    rc = library().bw_decode_step(ctypes.byref(a))
    if rc != SUCCESS:
        return rc, None
    engine._builder.mark_sent(ring)
    return rc, host
