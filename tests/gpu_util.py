"""Helpers shared by the GPU parity tests: hand a tests/synth.py model to the
CUDA provider (host pointers, uploaded once) and small torch<->pointer utilities."""
import ctypes as C

import numpy as np

from quantum_llm_b200 import lib as ql
from quantum_llm_b200.provider import Nvfp4MtpProvider, RequestParameters


def c_matrix(m):
    return ql.Matrix(m.codes.ctypes.data, m.scales.ctypes.data, float(m.weight_scale), float(m.input_scale),
                     m.rows, m.cols)


def c_block(b):
    if not getattr(b, "experts", 0):
        return ql.Block(b.input_norm.ctypes.data, c_matrix(b.qkv), c_matrix(b.o), b.post_norm.ctypes.data,
                        c_matrix(b.gate_up), c_matrix(b.down))
    arrays = [(ql.Matrix * b.experts)(*[c_matrix(m) for m in group])
              for group in (b.expert_gate, b.expert_up, b.expert_down)]
    b._c_arrays = arrays   # host arrays of expert descriptors: alive until the provider has copied them
    return ql.Block(b.input_norm.ctypes.data, c_matrix(b.qkv), c_matrix(b.o), b.post_norm.ctypes.data,
                    c_matrix(b.gate_up), c_matrix(b.down), c_matrix(b.router), arrays[0], arrays[1], arrays[2])


def c_config(cfg):
    c = ql.Config()
    for k, v in cfg.items():
        setattr(c, k, v)
    return c


def provider_from_synth(model, device=0):
    blocks = (ql.Block * len(model.layers))(*[c_block(b) for b in model.layers])
    w = ql.Weights(model.embedding.ctypes.data, blocks, model.final_norm.ctypes.data, c_matrix(model.head),
                   model.mtp_embedding_norm.ctypes.data, model.mtp_hidden_norm.ctypes.data,
                   c_matrix(model.mtp_fusion), c_block(model.mtp_block), model.mtp_draft_norm.ctypes.data)
    return Nvfp4MtpProvider(c_config(model.cfg), w, weights_on_device=False, device=device, keepalive=(model, blocks))


def request_pair(seed=1234, temperature_ppm=0, top_p_ppm=950000, top_k=20, min_p_ppm=0, context_limit=256,
                 presence_penalty_ppm=0, first_output_position=0):
    """The same request for the CUDA provider and for the oracle."""
    from tests import synth
    return (RequestParameters(seed, temperature_ppm, top_p_ppm, top_k, min_p_ppm, context_limit,
                              2_000_000 + presence_penalty_ppm, first_output_position),
            synth.request(seed, temperature_ppm, top_p_ppm, top_k, min_p_ppm, context_limit,
                          presence_penalty_ppm, first_output_position))


def dev(array):
    import torch
    return torch.from_numpy(np.ascontiguousarray(array)).cuda()


def bf16_ulps(a, b):
    """Distance in BF16 grid steps between two arrays of BF16-representable floats."""
    a = np.ascontiguousarray(a, np.float32).view(np.int32) >> 16
    b = np.ascontiguousarray(b, np.float32).view(np.int32) >> 16
    sa = np.where(a < 0, -(a & 0x7FFF), a)
    sb = np.where(b < 0, -(b & 0x7FFF), b)
    return np.abs(sa - sb)
