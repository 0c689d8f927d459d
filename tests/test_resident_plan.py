"""Plan and schedule of the slice-resident kernel, checked on the CPU through the library's diagnostic
exports: every piece of every channel is reduced once and applied once, in an order the shared-memory
slots can serve, and the roles of a block (loader, consumers, storer) cannot wait for one another in
a cycle.  No GPU is needed: the schedule is plain index arithmetic shared by host and device."""
import ctypes

import numpy as np
import pytest

from anode_b200 import _lib

RED_STR, RED_RES, PUBLISH, NEED_COEF, APP_STR, APP_RES = range(6)

SHAPES = [
    # dim0, C, N
    (3136, 256, 2048), (3136, 256, 1024), (3136, 256, 512), (3136, 256, 256), (12544, 64, 256),
    (2097152, 32, 4), (262144, 32, 4), (784, 64, 32), (196, 1024, 256), (784, 512, 32), (784, 16, 8),
    (3136, 8, 64), (3136, 16, 2048), (64, 3, 5), (4096, 1, 1), (1000, 7, 13), (68, 5, 300),
]


def plan(lib, d0, c, n, planes):
    out = (ctypes.c_uint32 * 16)()
    assert lib.anode_gpu_batch_norm_resident_plan(d0, c, n, planes, out) == 0
    keys = ("ok rpp P piece_len U Gt teams grid T slot_bytes Q Qr Qs Rz_max pf smem_bytes").split()
    return dict(zip(keys, list(out)))


def schedule(lib, d0, c, n, planes, block):
    cnt = lib.anode_gpu_batch_norm_resident_schedule(d0, c, n, planes, block, None, 0)
    assert cnt >= 0
    buf = (ctypes.c_uint32 * (4 * max(cnt, 1)))()
    assert lib.anode_gpu_batch_norm_resident_schedule(d0, c, n, planes, block, buf, cnt) == cnt
    return np.frombuffer(buf, dtype=np.uint32).reshape(-1, 4)[:cnt].copy()


def block_slice(p, block):
    b = block % p["Gt"]
    u0 = b * p["U"] // p["Gt"]
    u1 = (b + 1) * p["U"] // p["Gt"]
    return block // p["Gt"], u0, u1 - u0


def check_block(p, ev, block, channels):
    team, _, tb = block_slice(p, block)
    nchan = len(range(team, channels, p["teams"]))
    reduced, applied, published, coef = set(), set(), set(), set()
    for kind, k, piece, slot in ev.tolist():
        if kind in (RED_STR, RED_RES):
            assert (k, piece) not in reduced and k not in published
            assert slot < p["Qr"] if kind == RED_RES else p["Qr"] <= slot < p["Q"]
            reduced.add((k, piece))
        elif kind == PUBLISH:
            assert all((k, t) in reduced for t in range(tb)), "channel published before all of its pieces were reduced"
            published.add(k)
        elif kind == NEED_COEF:
            assert k in published
            coef.add(k)
        else:
            assert k in coef and (k, piece) in reduced and (k, piece) not in applied
            applied.add((k, piece))
    assert len(reduced) == len(applied) == nchan * tb and len(published) == nchan


def simulate(p, ev):
    """Three cursors over the same event list.  loader: issues the load of RED_* / APP_STR events when
    the slot is free; consumers: handle an event once its load (if any) was issued; storer: releases
    slots in order, keeping up to two stores' slots back unless it would have to wait."""
    ev = ev.tolist()
    n = len(ev)
    needs_load = [e[0] in (RED_STR, RED_RES, APP_STR) for e in ev]
    releases = [e[0] in (RED_STR, APP_STR, APP_RES) for e in ev]
    busy = [False] * p["Q"]
    li = ci = si = 0
    loaded = [False] * n
    pend = []
    steps = 0
    while ci < n or si < n:
        moved = False
        while li < n and not needs_load[li]:
            li += 1
        if li < n and not busy[ev[li][3]]:
            busy[ev[li][3]] = True
            loaded[li] = True
            li += 1
            moved = True
        if ci < n and (not needs_load[ci] or loaded[ci]):
            ci += 1
            moved = True
        while si < n and not releases[si]:
            si += 1
        if si < n:
            if si < ci:             # the consumers are done with this event
                kind, _, _, slot = ev[si]
                if kind == RED_STR:
                    busy[slot] = False
                else:
                    if len(pend) == 2:
                        busy[pend.pop(0)] = False
                    pend.append(slot)
                si += 1
                moved = True
            elif pend:              # about to wait: hand back what is held
                for s in pend:
                    busy[s] = False
                pend = []
                moved = True
        assert moved, "roles wait for one another: loader %d, consumers %d, storer %d of %d" % (li, ci, si, n)
        steps += 1
        assert steps < 20 * n + 100
    return True


@pytest.mark.parametrize("d0,c,n", SHAPES)
@pytest.mark.parametrize("planes", [1, 2, 3])
def test_schedule_is_complete_and_cannot_deadlock(d0, c, n, planes):
    lib = _lib.load()
    p = plan(lib, d0, c, n, planes)
    if not p["ok"]:
        pytest.skip("the slice-resident kernel does not take this shape")
    assert p["grid"] == p["Gt"] * p["teams"] <= 148 and p["teams"] <= c and p["Gt"] <= p["U"]
    assert p["Q"] == p["Qr"] + p["Qs"] <= 64 and p["smem_bytes"] <= 227 * 1024
    assert p["piece_len"] % 4 == 0 and p["rpp"] <= 32
    # the slices of a team tile the channel
    covered = 0
    for b in range(p["Gt"]):
        _, u0, tb = block_slice(p, b)
        assert u0 == covered and tb >= 1
        covered += tb
    assert covered == p["U"]
    for block in sorted({0, p["Gt"] - 1, p["grid"] - 1, p["grid"] // 2}):
        ev = schedule(lib, d0, c, n, planes, block)
        check_block(p, ev, block, c)
        simulate(p, ev)


def test_shapes_of_the_benchmark_are_taken():
    lib = _lib.load()
    for d0, c, n in SHAPES[:7]:
        for planes in (1, 2):
            assert plan(lib, d0, c, n, planes)["ok"], (d0, c, n, planes)
    assert not plan(lib, 49, 2048, 1024, 1)["ok"]      # rows that are not 16-byte multiples: the cluster kernel's shapes
