"""Device-side setup and one-step drivers for the benchmark workloads, on top of the C ABI (api.py).

torch is used for device memory, streams, events and the process group only; every computation is a call into
libosmos_b200.so.
"""
import numpy as np
import torch

from . import api, synth, workloads


def _dev_bytes(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


class MoeLane:
    """A routed-expert FFN layer (several cold copies of it) resident on one GPU, run through q4x_route + lane_ffn.

    expert_range (e0, e1): the experts this GPU owns (all of them on one GPU). Weights of the other experts are not
    uploaded; their addresses are never formed because no row of theirs exists in this GPU's tables.
    """

    def __init__(self, lib, cfg, dev, copies=1, max_tok=None, host_tensors=None, expert_range=None):
        self.lib, self.cfg, self.dev = lib, cfg, dev
        self.tid = synth.TYPE_ID[cfg["type"]]
        self.n_exp, self.k, self.dim, self.ff = cfg["n_exp"], cfg["k"], cfg["dim"], cfg["ff"]
        self.max_tok = max_tok or cfg["n_tok"]
        self.e0, self.e1 = expert_range or (0, self.n_exp)
        self.per = workloads.moe_expert_bytes(cfg)
        # host_tensors: the whole layer's, or (a workload whose experts have their own random streams) this range's only
        ranged = bool(cfg.get("per_expert_rng"))
        host = host_tensors or workloads.moe_layer_host(cfg, expert_range=(self.e0, self.e1) if ranged else None)
        self.host = host
        if ranged and host[0].size == (self.e1 - self.e0) * self.per[0]:
            first = [_dev_bytes(h, dev) for h in host]
        else:
            first = [_dev_bytes(h[self.e0 * b:self.e1 * b], dev) for h, b in zip(host, self.per)]
        self.weights = [first] + [[t.clone() for t in first] for _ in range(copies - 1)]
        self.layers = []
        for w in self.weights:
            layer = api.LaneLayer(self.tid, self.tid, self.dim, self.ff, self.n_exp, self.k, cfg["lim"], api.LaneExperts())
            for j in range(3):
                # base is where expert 0 would be: only experts e0 .. e1 are ever addressed
                layer.experts.base[j] = w[j].data_ptr() - self.e0 * self.per[j]
                layer.experts.bytes[j] = self.per[j]
            self.layers.append(layer)
        nbytes = lib.lane_scratch_bytes(self.layers[0], self.max_tok)
        assert nbytes, "lane_scratch_bytes refused the layer"
        self.scratch_mem = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
        self.scratch = api.LaneScratch()
        assert lib.lane_scratch_bind(self.layers[0], self.max_tok, self.scratch_mem.data_ptr(), nbytes, self.scratch)
        picks = self.max_tok * self.k
        self.ids = torch.zeros(picks, dtype=torch.int32, device=dev)
        self.wts = torch.zeros(picks, dtype=torch.float32, device=dev)
        self.rows = torch.zeros(picks, dtype=torch.int32, device=dev)
        self.kernels_per_step = 7  # route, tables (with the order), round, gate_up, round, down, sum

    def weight_bytes(self):
        return sum(t.numel() for t in self.weights[0])

    def step(self, x, logits, out, n_tok, copy=0, stream=0):
        """route + experts + combine for n_tok tokens; all tensors on the device. Raises if the ABI refuses."""
        lib = self.lib
        ok = lib.q4x_route(logits.data_ptr(), n_tok, self.n_exp, self.k, self.ids.data_ptr(), self.wts.data_ptr(),
                           self.rows.data_ptr(), stream)
        ok = ok and lib.lane_ffn(self.layers[copy % len(self.layers)], self.scratch, x.data_ptr(), self.ids.data_ptr(),
                                 self.wts.data_ptr(), n_tok, None, out.data_ptr(), stream)
        if not ok:
            raise RuntimeError("libosmos_b200 refused a call of the MoE step")

    def step_timed_gate_up(self, x, logits, out, n_tok, copy, ev0, ev1, stream=0):
        """the same step with the launches spelled out, CUDA events around the gate + up + activation kernel"""
        lib, s, L = self.lib, self.scratch, self.layers[copy % len(self.layers)]
        t = s.tab
        picks = n_tok * self.k
        ok = lib.q4x_route(logits.data_ptr(), n_tok, self.n_exp, self.k, self.ids.data_ptr(), self.wts.data_ptr(),
                           self.rows.data_ptr(), stream)
        ok = ok and lib.lane_tables(self.ids.data_ptr(), picks, self.k, self.n_exp, 0, self.n_exp, L.experts, t, stream)
        ok = ok and lib.q8_round(x.data_ptr(), n_tok, self.dim, self.dim, s.xq, s.xqd, stream)
        ev0.record()
        ok = ok and lib.q8_gate_up(self.tid, t.w[0], t.w[1], t.cnt, t.xrow, t.tok, t.pair, t.max_entries, 8, self.ff,
                                   self.dim, s.xq, s.xqd, self.wts.data_ptr(), self.cfg["lim"], s.hh, self.ff, stream)
        ev1.record()
        ok = ok and lib.q8_round(s.hh, picks, self.ff, self.ff, s.hq, s.hqd, stream)
        ok = ok and lib.q8_group_tok(self.tid, t.w[2], t.cnt, t.xrow, None, t.max_entries, 8, self.dim, self.ff, s.hq,
                                     s.hqd, s.ye, self.dim, stream)
        ok = ok and lib.ops_gather_sum(out.data_ptr(), s.ye, t.order, self.k, n_tok, self.dim, stream)
        if not ok:
            raise RuntimeError("libosmos_b200 refused a call of the MoE step")


def moe_oracle(oracle, cfg, host_tensors, x, ids, wts):
    """the layer's output by the CPU oracle: each pick's row through its expert, each token's rows added in ascending
    expert id (test / smoke use only)"""
    tid = synth.TYPE_ID[cfg["type"]]
    per = workloads.moe_expert_bytes(cfg)
    n_tok, dim, ff = x.shape[0], cfg["dim"], cfg["ff"]
    out = np.zeros((n_tok, dim), np.float32)
    for t in range(n_tok):
        acc = np.zeros(dim, np.float32)
        for j in np.argsort(ids[t], kind="stable"):
            e = int(ids[t, j])
            parts = [host_tensors[m][e * per[m]:(e + 1) * per[m]] for m in range(3)]
            y = oracle.lane_expert(tid, tid, parts[0], parts[1], parts[2], dim, ff, cfg["lim"], x[t:t + 1], wts[t, j:j + 1])
            acc = (acc + y[0]).astype(np.float32)
        out[t] = acc
    return out
