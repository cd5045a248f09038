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

# DeepSeek-V3-shape MoE decode layer: 256 IQ1_M experts of width 2048 over hidden 7168, top-8 by the scored router, and a
# Q4_K shared expert of the same three shapes on every token; 32 tokens a step, or 1
MOE_DS = dict(name="moe_iq1m_256e_top8_shared_q4k_b32", type="IQ1_M", n_exp=256, k=8, n_tok=32, dim=7168, ff=2048,
              sigma=0.01, lim=10.0, router="sqrt_softplus", route_scale=2.5, per_expert_rng=True,
              shared=dict(type="Q4_K", ff=2048, sigma=0.01, lim=10.0))
MOE_DS_B1 = dict(MOE_DS, name="moe_iq1m_256e_top8_shared_q4k_b1", n_tok=1)
# MXFP4 experts: 128 of gate / up [1536 x 4096], down [4096 x 1536], top-4; activations bf16 values; 32 tokens (decode, the
# F32 matvec over the experts) or 2048 (prefill, the grouped f16 product)
MOE_MX = dict(name="moe_mxfp4_128e_top4_b32", type="MXFP4", n_exp=128, k=4, n_tok=32, dim=4096, ff=1536, sigma=0.0,
              lim=7.0, per_expert_rng=True, bf16_inputs=True, path="f32_lane")
MOE_MX_PREFILL = dict(MOE_MX, name="moe_mxfp4_128e_top4_b2048", n_tok=2048, path="f16_group", lim=1.0e30)

# the prefill product with its rows split among the GPUs (a rank a slice of whole 128-row tiles, no collective)
DENSE_Q4_K = dict(MM_Q4_K, name="prefill_q4k_4096x4096_b512_rows", path="dense_rows")

BY_NAME = {c["name"]: c for c in (MOE_IQ3, MOE_DS, MOE_DS_B1, MOE_MX, MOE_MX_PREFILL, DENSE_Q4_K)}


def moe_layer_host(cfg, layer=0, expert_range=None):
    """the layer's three expert tensors (gate, up, down), each its experts one after another, as uint8 arrays; with
    expert_range (e0, e1) only those experts' bytes (a workload whose experts have their own random streams)"""
    tid = synth.TYPE_ID[cfg["type"]]
    if cfg.get("per_expert_rng"):
        e0, e1 = expert_range or (0, cfg["n_exp"])
        shapes = ((cfg["ff"], cfg["dim"]), (cfg["ff"], cfg["dim"]), (cfg["dim"], cfg["ff"]))
        out = []
        for m, (r, c) in enumerate(shapes):
            per = synth.tensor_bytes(tid, r, c)
            buf = np.empty((e1 - e0) * per, dtype=np.uint8)
            for e in range(e0, e1):
                buf[(e - e0) * per:(e - e0 + 1) * per] = synth.random_tensor(tid, r, c, synth.rng_for(303, tid, layer, m, e), cfg["sigma"])
            out.append(buf)
        return tuple(out)
    assert expert_range is None
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
    """a step's activations and router logits: F32 N(0,1) (bf16_inputs: the activations are bf16 values, held as F32)"""
    n_tok = n_tok or cfg["n_tok"]
    rng = synth.rng_for(302, step)
    x = rng.standard_normal((n_tok, cfg["dim"])).astype(np.float32)
    logits = rng.standard_normal((n_tok, cfg["n_exp"])).astype(np.float32)
    if cfg.get("bf16_inputs"):  # to the nearest bf16 (ties to even), as F32
        b = x.view(np.uint32)
        x = ((b + 0x7FFF + ((b >> 16) & 1)) & 0xFFFF0000).astype(np.uint32).view(np.float32)
    return x, logits


def shared_expert_host(cfg, layer=0):
    """the shared expert's three matrices (gate, up [ff x dim], down [dim x ff]) as uint8 arrays"""
    sh = cfg["shared"]
    tid = synth.TYPE_ID[sh["type"]]
    return tuple(synth.random_tensor(tid, r, c, synth.rng_for(304, tid, layer, m), sh["sigma"])
                 for m, (r, c) in enumerate(((sh["ff"], cfg["dim"]), (sh["ff"], cfg["dim"]), (cfg["dim"], sh["ff"]))))


def route_bias_host(cfg):
    return (synth.rng_for(305).standard_normal(cfg["n_exp"]) * 0.1).astype(np.float32)


def scored_topk(logits, bias, k, scale, kind="sqrt_softplus"):
    """ops_router's picks and weights in double precision: score = sqrt(softplus) or sigmoid, picked by score + bias (as
    F32 keys), w = score / sum of the picked scores * scale"""
    l = logits.astype(np.float64)
    sc = 1 / (1 + np.exp(-l)) if kind == "sigmoid" else np.sqrt(np.where(l > 20, l, np.log1p(np.exp(np.minimum(l, 20)))))
    key = (sc.astype(np.float32) + bias[None, :].astype(np.float32)).astype(np.float32)
    ids = np.argsort(-key, axis=1, kind="stable")[:, :k]
    pk = np.take_along_axis(sc, ids, 1)
    return ids.astype(np.int32), (pk / (pk.sum(1, keepdims=True) + 1e-20) * scale).astype(np.float32)


def route_host(cfg, logits):
    """the workload's router in double precision: (ids, weights)"""
    if cfg.get("router", "softmax") == "softmax":
        return softmax_topk(logits, cfg["k"])
    return scored_topk(logits, route_bias_host(cfg), cfg["k"], cfg["route_scale"], cfg["router"])


def softmax_topk(logits, k):
    """q4x_route's picks and weights in double precision (the ids are what the weights' bytes depend on)"""
    l = logits.astype(np.float64)
    p = np.exp(l - l.max(1, keepdims=True))
    p /= p.sum(1, keepdims=True)
    ids = np.argsort(-p, axis=1, kind="stable")[:, :k]
    pk = np.take_along_axis(p, ids, 1)
    return ids.astype(np.int32), (pk / np.maximum(pk.sum(1, keepdims=True), 2.0 ** -14)).astype(np.float32)


def router_check(cfg, logits, got_ids, got_wts, tol=2e-6):
    """whether a device's picks and weights are the workload's router's, in double precision: every picked key reaches the
    k-th greatest key (keys within `tol` of each other may be picked either way: the device's F32 scores round), the
    picks are distinct, in non-increasing key order (to `tol`), and the weights are the picked scores' normalisation"""
    l = logits.astype(np.float64)
    k = cfg["k"]
    if cfg.get("router", "softmax") == "softmax":
        p = np.exp(l - l.max(1, keepdims=True))
        key = score = p / p.sum(1, keepdims=True)
        norm = lambda pk: pk / np.maximum(pk.sum(1, keepdims=True), 2.0 ** -14)
    else:
        score = 1 / (1 + np.exp(-l)) if cfg["router"] == "sigmoid" else np.sqrt(np.where(l > 20, l, np.log1p(np.exp(np.minimum(l, 20)))))
        key = score + route_bias_host(cfg)[None, :].astype(np.float64)
        norm = lambda pk: pk / (pk.sum(1, keepdims=True) + 1e-20) * cfg["route_scale"]
    kth = -np.sort(-key, axis=1)[:, k - 1:k]
    gk = np.take_along_axis(key, got_ids.astype(np.int64), 1)
    scale = np.abs(key).max()
    distinct = all(len(set(r)) == k for r in got_ids.tolist())
    ordered = bool((gk[:, :-1] >= gk[:, 1:] - tol * scale).all()) if k > 1 else True
    reach = bool((gk >= kth - tol * scale).all())
    want_w = norm(np.take_along_axis(score, got_ids.astype(np.int64), 1))
    return distinct and ordered and reach and bool(np.allclose(got_wts, want_w, rtol=1e-5, atol=1e-12))
