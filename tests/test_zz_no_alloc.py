"""q4x_expert_tiles_static: the expert tables built with the library's own fixed scratch instead of a caller
buffer - for callers whose step path may not allocate device memory (a server running inside a start-up memory
budget, a plug-in whose host owns the allocator). Checked through the C ABI against q4x_expert_tiles on two calls
in a row that share the fixed array; exact equality (the tables are integers and addresses).

Collected last on purpose: a run that stops at the first failure has then run every other test already."""
import numpy as np
import pytest
import torch

from helpers import ptr, sync, to_dev
from libosmos_b200 import api, synth

pytestmark = pytest.mark.gpu

FIELDS = (("cnt", "entries"), ("gidx", "slots"), ("hidx", "slots"), ("xg", "entries"), ("yg", "entries"),
          ("xd", "entries"), ("yd", "entries"), ("where", "n"))


def _tables(lib, dev, n, n_exp, with_off):
    b = api.Q4xExpertBounds()
    lib.q4x_expert_bounds(n, n_exp, b)
    size = {"entries": b.entries, "slots": b.slots, "n": n}
    t, bufs = api.Q4xExpertTiles(), {}
    for j in range(3):
        t.base[j], t.bytes[j], t.tab[j] = 0x200000 * (j + 1), 1536 * (j + 1), None
        bufs["ptr%d" % j] = torch.zeros(b.entries, dtype=torch.int64, device=dev)
        t.ptr[j] = ptr(bufs["ptr%d" % j])
    for name, kind in FIELDS:
        bufs[name] = torch.full((size[kind],), 123, dtype=torch.int32, device=dev)
        setattr(t, name, ptr(bufs[name]))
    if with_off:
        bufs["off"] = torch.zeros(3 * n_exp, dtype=torch.int32, device=dev)
        t.off = ptr(bufs["off"])
    else:
        t.off = None  # the static variant ignores it
    return t, bufs


def test_static_scratch_matches_caller_scratch_twice(lib, dev):
    # (tokens, picks a token, experts): both above the 1024 picks the table kernel places itself, so the scratch is
    # what carries each expert's places from the first kernel to the second; the second call reuses the fixed array
    for call, (n_tok, k, n_exp) in enumerate([(700, 4, 16), (300, 8, 1024)]):
        rng = synth.rng_for(77, call)
        n, dim, ff = n_tok * k, 2048, 512
        ids = np.stack([rng.permutation(n_exp)[:k] for _ in range(n_tok)]).astype(np.int32).reshape(-1)
        ids_d = to_dev(ids, dev)
        t0, want = _tables(lib, dev, n, n_exp, with_off=True)
        t1, got = _tables(lib, dev, n, n_exp, with_off=False)
        assert lib.q4x_expert_tiles(ptr(ids_d), n, k, n_exp, dim, ff, t0, None)
        if call == 0:  # the first call on the device looks the array's address up: no allocation belongs to it either
            assert lib.q4x_expert_tiles_static(ptr(ids_d), n, k, n_exp, dim, ff, t1, None)
            sync()
        free_before = torch.cuda.mem_get_info()[0]
        assert lib.q4x_expert_tiles_static(ptr(ids_d), n, k, n_exp, dim, ff, t1, None)
        sync()
        assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the device's free memory"
        live = want["cnt"].cpu().numpy() > 0
        assert live.any()
        for name, _ in FIELDS:
            a, b_ = want[name].cpu().numpy(), got[name].cpu().numpy()
            if name in ("xg", "yg", "xd", "yd"):  # written for live entries only
                a, b_ = a[live], b_[live]
            assert np.array_equal(a, b_), name
        for j in range(3):
            assert np.array_equal(want["ptr%d" % j].cpu().numpy()[live], got["ptr%d" % j].cpu().numpy()[live])


def test_static_scratch_refuses_past_its_size(lib, dev):
    t, _ = _tables(lib, dev, 64, 16, with_off=False)
    ids = to_dev(np.zeros(64, np.int32), dev)
    assert not lib.q4x_expert_tiles_static(ptr(ids), 64, 4, 1025, 2048, 512, t, None)  # more experts than the array holds
    assert not lib.q4x_expert_tiles_static(ptr(ids), 64, 4, 0, 2048, 512, t, None)
    assert not lib.q4x_expert_tiles_static(ptr(ids), 64, 4, 16, 2048, 512, None, None)
