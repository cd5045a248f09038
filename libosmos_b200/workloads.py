"""The benchmark configurations as seeded synthetic workloads (host-side construction shared by bench.py, the smoke
check and the full-size GPU tests). No model files exist here, so tensors are synthetic blocks with the
configurations' recipes (see synth.py).
"""
import numpy as np

from . import synth

# Qwen-style MoE FFN layer in IQ3_XXS: 512 experts, top-10 of 64 tokens, hidden 2048, expert width 512
MOE_IQ3 = dict(name="moe_iq3xxs_512e_top10", type="IQ3_XXS", n_exp=512, k=10, n_tok=64, dim=2048, ff=512,
               sigma=0.005, lim=1.0e30)
# the decode matvec: Q4_0 W[6144 x 2048], one token
MV_Q4_0 = dict(name="mv_q4_0_6144x2048", type="Q4_0", rows=6144, cols=2048, sigma=0.01)
# the prefill product: Q4_K W[4096 x 4096] over 512 tokens
MM_Q4_K = dict(name="mm_q4_k_4096x4096x512", type="Q4_K", rows=4096, cols=4096, tokens=512, sigma=0.01)

BY_NAME = {MOE_IQ3["name"]: MOE_IQ3}


def moe_layer_host(cfg, layer=0):
    """the layer's three expert tensors (gate, up, down), each its experts one after another, as uint8 arrays"""
    tid = synth.TYPE_ID[cfg["type"]]
    rng = synth.rng_for(301, tid, layer)
    gate = synth.random_tensor(tid, cfg["n_exp"] * cfg["ff"], cfg["dim"], rng, cfg["sigma"])
    up = synth.random_tensor(tid, cfg["n_exp"] * cfg["ff"], cfg["dim"], rng, cfg["sigma"])
    down = synth.random_tensor(tid, cfg["n_exp"] * cfg["dim"], cfg["ff"], rng, cfg["sigma"])
    return gate, up, down


def moe_expert_bytes(cfg):
    tid = synth.TYPE_ID[cfg["type"]]
    gu = synth.tensor_bytes(tid, cfg["ff"], cfg["dim"])
    return gu, gu, synth.tensor_bytes(tid, cfg["dim"], cfg["ff"])


def moe_inputs_host(cfg, step=0, n_tok=None):
    """a step's activations and router logits: F32 N(0,1)"""
    n_tok = n_tok or cfg["n_tok"]
    rng = synth.rng_for(302, step)
    x = rng.standard_normal((n_tok, cfg["dim"])).astype(np.float32)
    logits = rng.standard_normal((n_tok, cfg["n_exp"])).astype(np.float32)
    return x, logits


def softmax_topk(logits, k):
    """q4x_route's picks and weights in double precision (the ids are what the weights' bytes depend on)"""
    l = logits.astype(np.float64)
    p = np.exp(l - l.max(1, keepdims=True))
    p /= p.sum(1, keepdims=True)
    ids = np.argsort(-p, axis=1, kind="stable")[:, :k]
    pk = np.take_along_axis(p, ids, 1)
    return ids.astype(np.int32), (pk / np.maximum(pk.sum(1, keepdims=True), 2.0 ** -14)).astype(np.float32)
