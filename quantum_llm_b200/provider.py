"""Python mirror of the reference's exact-decode provider interface
(expert::runtime::IOperationProvider, runtime/include/expert/runtime/program_executor.hpp:244-370)
over the C ABI.  Method names, argument meaning and failure behaviour follow the
reference: every call either succeeds or raises QllmError carrying the status
code that the reference would return in its Status.
"""
import ctypes as C
from dataclasses import dataclass, field
from typing import List

import numpy as np

from . import lib as _l


@dataclass
class RequestParameters:
    """ProgramRequestContext.parameters read on the exact-decode path
    (runtime/tools/moe_vm_runner.cpp:318-347)."""
    sampling_seed: int = 0
    sampling_temperature_ppm: int = 0
    sampling_top_p_ppm: int = 1_000_000
    sampling_top_k: int = 20
    sampling_min_p_ppm: int = 0
    reserved_context_tokens: int = 0
    sampling_presence_penalty_biased_ppm: int = 2_000_000   # penalty * 1e6 + 2e6; 2e6 = none, at most 4e6
    sampling_first_output_position: int = 0                 # the scalar head penalises and marks from here on

    def c(self):
        return _l.Request(self.sampling_seed, self.sampling_temperature_ppm, self.sampling_top_p_ppm,
                          self.sampling_top_k, self.sampling_min_p_ppm, self.reserved_context_tokens,
                          self.sampling_presence_penalty_biased_ppm, self.sampling_first_output_position, 0)


@dataclass
class ExactDecodeResult:
    """ExactDecodeExecutionResult (program_executor.hpp:205-212)."""
    emitted_tokens: List[int] = field(default_factory=list)
    next_token: int = 0
    positions_advanced: int = 0
    rejected: bool = False


def _result(r):
    return ExactDecodeResult([int(t) for t in r.emitted_tokens[:r.emitted_count]], int(r.next_token),
                             int(r.positions_advanced), bool(r.rejected))


class RequestState:
    def __init__(self, provider):
        self.provider = provider
        h = C.c_void_p()
        _l.check(provider.L.qllm_provider_create_request_state(provider.h, C.byref(h)))
        self.h = h

    def close(self):
        if self.h:
            self.provider.L.qllm_provider_destroy_request_state(self.provider.h, self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Nvfp4MtpProvider:
    """Drop-in for DenseFp4Provider's exact-decode service on NVFP4 weights.

    `config` is a lib.Config, `weights` a lib.Weights whose pointers are device
    addresses (weights_on_device=True, borrowed) or host addresses (uploaded once).
    """

    MAX_ROWS = 8

    def __init__(self, config, weights, weights_on_device, device=0, keepalive=None):
        self.L = _l.load()
        self.config = config
        self._keep = (config, weights, keepalive)
        h = C.c_void_p()
        _l.check(self.L.qllm_provider_create(C.byref(config), C.byref(weights), int(weights_on_device), device,
                                            C.byref(h)))
        self.h = h

    def close(self):
        if self.h:
            self.L.qllm_provider_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @staticmethod
    def capability():
        L = _l.load()
        return L.qllm_capability_name().decode(), int(L.qllm_capability_abi())

    # -- IOperationProvider ---------------------------------------------------
    def create_request_state(self):
        return RequestState(self)

    def prefill_chunk(self, state, tokens, first_position):
        tokens = np.ascontiguousarray(tokens, np.uint32)
        _l.check(self.L.qllm_provider_prefill_chunk(self.h, state.h, tokens.ctypes.data, len(tokens), first_position))

    def first_token(self, state, request, sample_position):
        token = C.c_uint32(0)
        rq = request.c()
        _l.check(self.L.qllm_provider_first_token(self.h, state.h, C.byref(rq), sample_position, C.byref(token)))
        return token.value

    def scalar_decode(self, state, request, token, position, produce_final_draft=False):
        """One non-speculative step: `token` at `position` through the target, next token by the
        request's sampler (any top_k), draft cache advanced by a one-row synchronisation batch."""
        nxt = C.c_uint32(0)
        rq = request.c()
        _l.check(self.L.qllm_provider_scalar_decode(self.h, state.h, C.byref(rq), token, position,
                                                    1 if produce_final_draft else 0, C.byref(nxt)))
        return nxt.value

    def checkpoint_request_state(self, state, next_position):
        _l.check(self.L.qllm_provider_checkpoint_request_state(self.h, state.h, next_position))

    def rewind_request_state(self, state, next_position):
        _l.check(self.L.qllm_provider_rewind_request_state(self.h, state.h, next_position))

    def synchronize_exact_decode_batch(self, state, request, next_tokens, first_target_position,
                                       produce_final_draft):
        next_tokens = np.ascontiguousarray(next_tokens, np.uint32)
        rq = request.c()
        _l.check(self.L.qllm_provider_synchronize_exact_decode_batch(
            self.h, state.h, C.byref(rq), next_tokens.ctypes.data, len(next_tokens), first_target_position,
            int(produce_final_draft)))

    def execute_exact_decode(self, state, request, guaranteed_token, position, context_limit):
        rq = request.c()
        res = _l.ExactResult()
        _l.check(self.L.qllm_provider_execute_exact_decode(self.h, state.h, C.byref(rq), guaranteed_token, position,
                                                          context_limit, C.byref(res)))
        return _result(res)

    def execute_exact_decode_steps(self, state, request, context_limit, steps):
        rq = request.c()
        res = (_l.ExactResult * steps)()
        _l.check(self.L.qllm_provider_execute_exact_decode_steps(self.h, state.h, C.byref(rq), context_limit, steps, res))
        return [_result(r) for r in res]

    # -- convenience over the reference's call order ----------------------------
    def prefill(self, state, request, tokens, first_position=0, chunk_rows=5):
        """Runner sequence of moe_vm_runner.cpp:679-778: target chunks, then the
        synchronisation batch of each chunk; returns the first generated token."""
        tokens = np.ascontiguousarray(tokens, np.uint32)
        count = len(tokens)
        first_token = None
        for first in range(0, count, chunk_rows):
            rows = min(chunk_rows, count - first)
            last = first + rows == count
            self.prefill_chunk(state, tokens[first:first + rows], first_position + first)
            if last:
                first_token = self.first_token(state, request, first_position + count - 1)
            nxt = np.empty(rows, np.uint32)
            nxt[:rows - 1] = tokens[first + 1:first + rows]
            nxt[rows - 1] = tokens[first + rows] if not last else first_token
            self.synchronize_exact_decode_batch(state, request, nxt, first_position + first, last)
        return first_token

    # -- settings / inspection ---------------------------------------------------
    def stream(self):
        """The provider's cudaStream_t as an integer handle."""
        return int(self.L.qllm_provider_stream(self.h) or 0)

    def max_chunk_rows(self):
        """Most rows one prefill chunk / synchronisation batch may hold."""
        return int(self.L.qllm_provider_max_chunk_rows(self.h))

    def set_graph_mode(self, enabled):
        _l.check(self.L.qllm_provider_set_graph_mode(self.h, int(enabled)))

    def set_attention_impl(self, impl):
        _l.check(self.L.qllm_provider_set_attention_impl(self.h, int(impl)))

    def tp_export(self, rank, ranks):
        """Allocates this rank's tensor-parallel exchange area; returns its inter-process handle."""
        handle = C.create_string_buffer(_l.TP_HANDLE_BYTES)
        _l.check(self.L.qllm_provider_tp_export(self.h, int(rank), int(ranks), handle))
        return handle.raw

    def tp_attach(self, handles):
        """Maps the peers' exchange areas: `handles` = the ranks' handles concatenated in rank order."""
        buffer = C.create_string_buffer(bytes(handles), len(handles))
        _l.check(self.L.qllm_provider_tp_attach(self.h, buffer))

    def tp_area_bytes(self):
        return int(self.L.qllm_provider_tp_area_bytes(self.h))

    def tp_attach_local(self, areas):
        """`areas[r]`: device pointer of rank r's exchange area (one process driving all GPUs)."""
        table = (C.c_void_p * len(areas))(*[C.c_void_p(a) for a in areas])
        _l.check(self.L.qllm_provider_tp_attach_local(self.h, table))

    def set_gemv_impl(self, impl):
        _l.check(self.L.qllm_provider_set_gemv_impl(self.h, int(impl)))

    def telemetry(self, state):
        out = (C.c_uint64 * 8)()
        _l.check(self.L.qllm_provider_telemetry(self.h, state.h, out, 8))
        v = [int(x) for x in out]
        return {"exact_calls": v[0], "accepted_drafts": v[1], "accepted_depth_calls": v[2:7], "kernel_launches": v[7]}

    def read_logits(self, rows):
        out = np.empty((rows, self.config.vocab), np.float32)
        _l.check(self.L.qllm_provider_read_logits(self.h, out.ctypes.data, rows))
        return out

    def read_hidden(self, state, which, rows):
        out = np.empty((rows, self.config.hidden), np.float32)
        _l.check(self.L.qllm_provider_read_hidden(self.h, state.h, which, out.ctypes.data, rows))
        return out

    def read_drafts(self, state):
        toks = np.zeros(4, np.uint32)
        n = C.c_uint32(0)
        _l.check(self.L.qllm_provider_read_drafts(self.h, state.h, toks.ctypes.data, C.byref(n)))
        return toks[:n.value].copy()

    def page_bytes(self):
        return self.L.qllm_provider_page_bytes(self.h)

    def layer_offset(self, layer):
        return self.L.qllm_provider_layer_offset(self.h, layer)

    def read_page(self, state, page):
        out = np.empty(self.page_bytes(), np.uint8)
        _l.check(self.L.qllm_provider_read_page(self.h, state.h, page, out.ctypes.data))
        return out

    def time_verify(self, state, request, repeats=8):
        """Mean duration (ms, CUDA events) of the verify pass alone over the pending drafts."""
        ms = C.c_float(0.0)
        rq = request.c()
        _l.check(self.L.qllm_provider_time_verify(self.h, state.h, C.byref(rq), repeats, C.byref(ms)))
        return ms.value

    def fill_synthetic_kv(self, state, first, count, seed):
        _l.check(self.L.qllm_provider_fill_synthetic_kv(self.h, state.h, first, count, seed))
