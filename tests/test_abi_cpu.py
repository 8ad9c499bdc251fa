"""The C-ABI library on a machine without a GPU: it loads, exports every declared symbol and rejects
bad arguments on the host with the documented codes (no kernel is launched here)."""

from __future__ import annotations

import ctypes
import os
import re

import pytest
import torch

from sparse_kv_reads_b200 import _lib
from sparse_kv_reads_b200.build import build
from sparse_kv_reads_b200.cluster_state import ClusterArena, SphereIndexGraph

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L():
    build()
    return _lib.lib()


def declared_functions():
    text = open(os.path.join(ROOT, "include", "skv.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(skv_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_entry_point_is_exported(L):
    names = declared_functions()
    assert len(names) >= 13
    for name in names:
        assert hasattr(L, name), name
    assert set(names) == set(_lib.EXPORTS)
    assert L.skv_version() == 101
    assert L.skv_error_string(-4).decode().startswith("pointer or stride")


def test_struct_layout_matches_the_header():
    text = open(os.path.join(ROOT, "include", "skv.h")).read()
    body = text[text.index("typedef struct skv_state {"):text.index("} skv_state;")]
    fields = re.findall(r"^\s+(?:int32_t|float|int8_t|int16_t)\s+\*?([A-Za-z0-9_]+);", body, flags=re.M)
    assert fields == [f[0] for f in _lib.SkvState._fields_]
    assert ctypes.sizeof(_lib.SkvState) == 6 * 4 + 19 * 8


def fake_state(C=64, cap=64, bits=32, heads=2):
    """A state whose pointers are aligned non-null fakes: validation must reject before use."""
    s = _lib.SkvState()
    s.heads, s.C, s.d, s.capacity, s.summary_bits = heads, C, 128, cap, bits
    for name, _ in _lib.SkvState._fields_[6:]:
        setattr(s, name, 0x1000)
    return s


def test_attend_rejects_bad_arguments(L):
    ok = 0x1000
    args = dict(q=ok, K=ok, V=ok, idx=ok, cnt=ok, n_dev=None, out=ok, ws=ok, status=None, heads=2, G=2, d=128, dtype=0,
                ksh=128 * 64, ksr=128, vsh=128 * 64, vsr=128, istr=64, lim=64, splits=4)

    def call(**over):
        a = {**args, **over}
        return L.skv_attend(a["q"], a["K"], a["V"], a["idx"], a["cnt"], a["n_dev"], 0, a["out"], a["ws"], a["status"],
                            a["heads"], a["G"], a["d"], a["dtype"], a["ksh"], a["ksr"], a["vsh"], a["vsr"], a["istr"],
                            a["lim"], a["splits"], 0.1, None)

    assert call(q=None) == -1 and call(cnt=None) == -1 and call(idx=None, n_dev=None) == -1
    assert call(d=64) == -2 and call(G=17) == -2 and call(dtype=1, G=9) == -2
    assert call(dtype=7) == -3
    assert call(K=0x1008) == -4 and call(ksr=100) == -4 and call(ksr=132) == -4
    assert call(heads=0) == -5 and call(splits=0) == -5
    assert L.skv_attend_splits(8) == 37 and L.skv_attend_splits(0) == -5        # one wave of 148 SMs
    assert L.skv_attend_splits(64) == 6 and L.skv_attend_splits(256) == 1 and L.skv_attend_splits(1000) == 1
    assert L.skv_attend_workspace_bytes(8, 2, 128, 37) == 8 * 37 * 2 * 132 * 4 + 256
    assert L.skv_attend_workspace_bytes(8, 2, 64, 37) == -5


def test_attend_static_rejects_the_same_calls_before_any_cuda_call(L):
    """The no-allocation entry point validates like skv_attend and checks its size limit on the host: on a
    machine without a GPU every rejected call returns its argument code, never SKV_E_CUDA."""
    ok = 0x1000
    args = dict(q=ok, K=ok, V=ok, idx=ok, cnt=ok, n_dev=None, out=ok, status=None, heads=2, G=2, d=128, dtype=0,
                ksh=128 * 64, ksr=128, vsh=128 * 64, vsr=128, istr=64, lim=64, splits=4)

    def call(**over):
        a = {**args, **over}
        return L.skv_attend_static(a["q"], a["K"], a["V"], a["idx"], a["cnt"], a["n_dev"], 0, a["out"], a["status"],
                                   a["heads"], a["G"], a["d"], a["dtype"], a["ksh"], a["ksr"], a["vsh"], a["vsr"],
                                   a["istr"], a["lim"], a["splits"], 0.1, None)

    assert call(q=None) == -1 and call(cnt=None) == -1 and call(idx=None, n_dev=None) == -1
    assert call(d=64) == -2 and call(G=17) == -2
    assert call(dtype=7) == -3
    assert call(K=0x1008) == -4 and call(ksr=100) == -4
    assert call(heads=0) == -5 and call(splits=0) == -5
    assert call(heads=4096, G=8, splits=64) == -8
    assert L.skv_attend_workspace_bytes(4096, 8, 128, 64) > 8 * 1024 * 1024
    assert L.skv_error_string(-8).decode().startswith("request exceeds")


def test_state_calls_reject_bad_arguments(L):
    ok = 0x1000
    st = fake_state()
    sel = lambda s, **o: L.skv_select(ctypes.byref(s), o.get("q", ok), o.get("dtype", 0), o.get("G", 2), ok, o.get("ng", 0), ok, ok,
                                      ok, o.get("istr", 64), ok, None, None, None, o.get("ws", ok), 0.1, o.get("group", 0),
                                      o.get("rope", None), None)
    assert sel(fake_state(C=48)) == -2 and sel(fake_state(C=8)) == -2 and sel(st, G=0) == -2
    assert sel(st, q=None) == -1 and sel(st, dtype=5) == -3 and sel(st, istr=8) == -5
    assert sel(st, group=3) == -5 and sel(st, group=-1) == -5 and sel(st, ng=-1) == -5
    assert sel(fake_state(cap=60)) == -4 and sel(fake_state(bits=16)) == -5
    bad = fake_state(bits=8)
    bad.dir8 = None
    assert sel(bad) == -1 and sel(st, ws=None) == -1
    assert L.skv_select_workspace_bytes(8, 2, 2048) == 8 * 2 * 2048 * 4 + 256 + 2304 + 8 * 64 * 32 * 4
    assert L.skv_select_workspace_bytes(8, 2, 100) == -5
    lab = lambda **o: L.skv_attend_labels(ok, ok, ok, ok, o.get("ls", 64), ok, o.get("C", 64), ok, o.get("ng", 0), ok, ok,
                                          None, None, 2,
                                          o.get("G", 2), 128, o.get("dtype", 0), 128 * 64, 128, 128 * 64, 128, 4, 0.1, None)
    assert lab(ng=-2) == -5
    assert lab(ls=36) == -4 and lab(C=48) == -2 and lab(dtype=1) == -3 and lab(G=17) == -2
    ins = lambda s, **o: L.skv_insert(ctypes.byref(s), ok, o.get("hpl", 2), 0, 128 * 64, o.get("ksr", 128), ok, o.get("ng", 0), 64,
                                      0.2, 0.03, o.get("reset_at", 0), o.get("mm", 66), o.get("capk", 0.0),
                                      o.get("var_min", 8), None)
    assert ins(st, hpl=3) == -5 and ins(st, mm=1) == -5 and ins(st, mm=10 ** 6) == -5 and ins(st, ksr=120) == -4
    assert ins(st, capk=-1.0) == -5 and ins(st, var_min=-1) == -5 and ins(st, reset_at=-1) == -5 and ins(st, ng=-1) == -5
    assert L.skv_insert_max_members() >= 400
    fit = lambda s, **o: L.skv_fit(ctypes.byref(s), ok, 0, 128 * 64, 128, o.get("n", 64), o.get("window", 8),
                                   o.get("C_init", 16), 10, ok, 0.0, 0.0, o.get("capk", 0.0), o.get("vf", 0.0),
                                   o.get("hl", None), o.get("nl", 0), o.get("kl", None), o.get("hpl", 0), ok,
                                   o.get("bytes", 1 << 40), None)
    assert fit(st, n=100) == -5 and fit(st, C_init=128) == -5 and fit(st, n=8, window=8) == -5
    assert fit(st, kl=ok, hpl=3) == -5 and fit(st, kl=ok, hpl=0) == -5      # heads of st must divide into layers
    assert fit(st, capk=-1.0) == -5 and fit(st, vf=-0.5) == -5 and fit(st, hl=ok, nl=0) == -5 and fit(st, hl=ok, nl=3) == -5
    assert fit(st, bytes=16) == -6
    assert L.skv_fit_workspace_bytes(2, 55, 64, 128) > 2 * 55 * 512
    assert L.skv_rebin(ctypes.byref(st), ok, 3, 32, ok, 0, 128 * 64, 128, 0.0, 10, 0.0, ok, 1 << 40, None) == -5
    assert L.skv_merge(None, ok, ok, ok, 1, 1, 1, 128, None) == -1


def test_host_class_options_follow_the_reference():
    with pytest.raises(ValueError):
        SphereIndexGraph(partition="spiral")
    with pytest.raises(ValueError):
        SphereIndexGraph(summary_bits=16)
    with pytest.raises(ValueError):
        SphereIndexGraph(C=64, C_init=128)
    with pytest.raises(AssertionError):
        SphereIndexGraph(C=48)
    ix = SphereIndexGraph(C=1024, C_init=256, cap_keys=64.0)
    assert ix.split_factor == 2.0 and ix.splitting                   # an absolute cap turns splitting on
    assert not SphereIndexGraph(C=256).splitting
    arena = ClusterArena(layers=3, h=2, C=16, d=128, capacity=64, summary_bits=8, device=torch.device("cpu"))
    v = arena.views(1)
    assert v["labels"].shape == (2, 64) and int(v["labels"][0, 0]) == 16 and torch.isinf(v["mmin"]).all()
    s = arena.struct(2, 4)
    assert s.heads == 2 and s.labels == arena.t["labels"][2:4].data_ptr()
    with pytest.raises(ValueError):
        ClusterArena(layers=1, h=1, C=16, d=128, capacity=60, summary_bits=8, device=torch.device("cpu"))


def test_a_missing_library_is_a_loud_error(monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libskv.so")
    with pytest.raises(_lib.SkvError):
        _lib.lib()


def test_state_dict_round_trip_on_the_cpu():
    """Checkpoint / resume of one layer's cluster state: arrays and counters survive a save and a load."""
    dev = torch.device("cpu")
    a = SphereIndexGraph(C=16, window=4, capacity=64, summary_bits=8)
    with pytest.raises(ValueError):
        a.state_dict()
    a._alloc(2, 128, dev)
    a.sum_dir.normal_()
    a.count.fill_(3.0)
    a.n_c.fill_(7)
    a.labels[:, 1:20] = 5
    a.end_dev.fill_(20)
    a.initialized, a._fitted, a.n, a.rebuilds, a._steps = True, True, 24, 2, 9
    sd = a.state_dict()
    assert sd["host"]["end"] == 20 and sd["arrays"]["labels"].dtype == torch.int16
    b = SphereIndexGraph(C=16, window=4, capacity=64, summary_bits=8)
    b.load_state_dict(sd, dev)
    for name in ("sum_dir", "count", "n_c", "labels", "dir8", "end_dev"):
        assert torch.equal(getattr(a, name), getattr(b, name)), name
    assert (b.n, b.end, b.rebuilds, b._steps, b.initialized) == (24, 20, 2, 9, True)
    with pytest.raises(ValueError):
        SphereIndexGraph(C=32, window=4, capacity=64).load_state_dict(sd, dev)
    from sparse_kv_reads_b200.stamp import stamp
    assert {"time", "host_cores", "torch"} <= set(stamp())


def test_matrix_vector_product_and_exchange_reject_bad_arguments(L):
    ok = 0x1000
    gemv = lambda **o: L.skv_gemv(o.get("W", ok), o.get("N", 64), o.get("K", 128), o.get("y", ok), o.get("B", 1),
                                  o.get("mode", 0), o.get("x", ok), o.get("h_in", None), None, o.get("g", None), None,
                                  1e-6, None)
    assert gemv(W=None) == -1 and gemv(y=None) == -1 and gemv(x=None) == -1
    assert gemv(mode=1) == -1                              # residual add + norm needs h_in and the norm weights
    assert gemv(mode=3) == -5 and gemv(mode=7) == -5       # mode 3 only through skv_gemv_tp
    assert gemv(B=0) == -5 and gemv(B=9) == -5 and gemv(K=12) == -5 and gemv(N=0) == -5
    assert gemv(W=0x1008) == -4 and gemv(x=0x1004) == -4
    assert L.skv_gemv_supported(64, 12, 1, 0) == 0 and L.skv_gemv_supported(64, 128, 9, 0) == 0
    # exchange buffers: sizes and the regions of a view
    assert L.skv_comm_bytes(0, 1024) == -5 and L.skv_comm_bytes(9, 1024) == -5 and L.skv_comm_bytes(2, 12) == -5
    assert L.skv_comm_bytes(2, 1024) == 2 * 2 * 1024 * 8 + 256
    bases = (ctypes.c_void_p * 2)(0x10000, 0x90000)
    c = _lib.SkvComm()
    assert L.skv_comm_view(ctypes.byref(c), bases, 2, 1, 1024) == 0
    assert (c.world, c.rank, c.cap_elems) == (2, 1, 1024)
    assert c.data[0] == 0x10000 and c.data[1] == 0x90000
    assert c.tick == 0x90000 + 2 * 2 * 1024 * 8 and c.status == c.tick + 64
    assert L.skv_comm_view(ctypes.byref(c), bases, 2, 2, 1024) == -5
    assert L.skv_comm_view(None, bases, 2, 0, 1024) == -1
    tp = lambda **o: L.skv_gemv_tp(ok, 64, 128, o.get("y", None), 1, o.get("mode", 0), ok, ok, ok, None, 1e-6,
                                   o.get("cin", None), o.get("in_seq", 0), o.get("cout", None), o.get("out_seq", 0), None)
    assert tp() == -1                                      # neither y nor an exchange to deliver to
    assert tp(mode=3, y=ok) == -5 and tp(cin=ctypes.byref(c), y=ok) == -5     # mode 3 <=> an exchange to read from
    assert tp(cout=ctypes.byref(c), out_seq=255) == -5 and tp(mode=3, cin=ctypes.byref(c), in_seq=-1, y=ok) == -5
    assert L.skv_comm_reduce(None, 0, ok, 1, 128, None) == -1
    assert L.skv_comm_reduce(ctypes.byref(c), 0, ok, 1, 12, None) == -5
    assert L.skv_comm_push(None, 0, ok, 1, 128, None) == -1 and L.skv_comm_push(ctypes.byref(c), 0, None, 1, 128, None) == -1
    assert L.skv_comm_push(ctypes.byref(c), 0, ok, 1, 12, None) == -5 and L.skv_comm_push(ctypes.byref(c), 255, ok, 1, 128, None) == -5
    assert L.skv_comm_push(ctypes.byref(c), 0, ok, 9, 128, None) == -5        # more than the buffers hold
    assert L.skv_comm_push(ctypes.byref(c), 0, 0x1004, 1, 128, None) == -4
    assert L.skv_comm_tick(None, None) == -1


def test_header_is_plain_c(tmp_path):
    """include/skv.h compiles as C99 with no framework headers: what a cgo / JNI / FFI binding needs."""
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    src = tmp_path / "use.c"
    src.write_text('#include <stddef.h>\n#include "skv.h"\n'
                   "int main(void) { skv_state s; skv_comm c; skv_rope r; (void)s; (void)c; (void)r;\n"
                   "  return skv_version() == SKV_VERSION ? 0 : 1; }\n")
    subprocess.check_call([gcc, "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-I",
                           os.path.join(ROOT, "include"), "-c", str(src), "-o", str(tmp_path / "use.o")])


def test_weighted_attention_rejects_bad_arguments(L):
    ok = 0x1000

    def call(**over):
        a = dict(q=ok, K=ok, V=ok, labels=ok, lstr=64, w=ok, C=64, n_dev=ok, out=ok, ws=ok, heads=2, G=2, d=128, dtype=0,
                 ksr=128, splits=4)
        a.update(over)
        return L.skv_attend_weighted(a["q"], a["K"], a["V"], a["labels"], a["lstr"], a["w"], a["C"], a["n_dev"], 0,
                                     a["out"], a["ws"], None, a["heads"], a["G"], a["d"], a["dtype"], 128 * 64, a["ksr"],
                                     128 * 64, 128, a["splits"], 0.1, None)

    assert call(labels=None) == -1 and call(w=None) == -1 and call(n_dev=None) == -1
    assert call(G=9) == -2 and call(C=48) == -2 and call(d=64) == -2
    assert call(dtype=5) == -3 and call(ksr=100) == -4 and call(lstr=0) == -5 and call(splits=0) == -5


def test_one_launch_step_rejects_bad_arguments(L):
    st = fake_state(C=256, cap=4096, bits=8, heads=8)
    ok = 0x1000

    def call(state=st, **over):
        a = dict(q=ok, G=2, n_dev=ok, K=ok, V=ok, ksr=128, cnt=ok, out=ok, ws=ok, clusters=4)
        a.update(over)
        return L.skv_step(ctypes.byref(state), a["q"], a["G"], a["n_dev"], a.get("ng", 0), a["K"], a["V"], 128 * 4096,
                          a["ksr"],
                          128 * 4096, 128, None, None, a["cnt"], a["out"], a["ws"], a["clusters"], 0.1, None, None)

    assert call(q=None) == -1 and call(K=None) == -1 and call(ws=None) == -1
    assert call(G=9) == -2 and call(clusters=9) == -2
    assert call(state=fake_state(C=4096, cap=4096, bits=8, heads=8)) == -2        # more than 2,048 slots
    assert call(state=fake_state(C=256, cap=4096, bits=32, heads=8)) in (-1, -5)  # float32 summaries: not served
    assert call(ksr=100) == -4 and call(clusters=0) == -5
    assert L.skv_step_workspace_bytes(8, 2, 4) == 8 * 4 * 2 * 132 * 4 + 256
    assert L.skv_step_clusters(8, 2, 4096, 8) == 0 and L.skv_step_clusters(8, 2, 256, 32) == 0
    assert L.skv_gemv_attended(ok, 64, 256, ok, 1, None, 4, 2, None, None, 0, None) == -1
    assert L.skv_gemv_attended(ok, 64, 256, ok, 1, ok, 9, 2, None, None, 0, None) == -5
