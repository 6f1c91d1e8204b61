"""Host-side pieces of layer-list models: the config reader and the scheduler's state slots and scripted steps."""
import ctypes as C
import json

import numpy as np

from oracle import hybrid as oh


def test_config_reader_takes_every_size_from_config(kge, tmp_path):
    cfg = oh.make_config(vocab=131, width=40, layers=("rglru", "parallel", "parallel"), mlps=("moe-noshared", None, "dense"),
                         heads=6, kv_heads=3, dim=10, vdim=14, chunk=17, m_heads=2, m_dim=6, m_vdim=12, r_width=60, r_blocks=5,
                         r_conv=2, ff=50, experts=7, top=3, expert_ff=9)
    oh.save_model_dir(str(tmp_path), cfg, oh.make_weights(cfg))
    L = kge.lib()
    h = L.kge_model_open(str(tmp_path).encode())
    assert h, L.kge_last_error()
    buf = C.create_string_buffer(8192)
    assert L.kge_model_spec_json(h, buf, 8192) > 0
    spec = json.loads(buf.value)
    L.kge_model_close(h)
    assert (spec["vocab"], spec["d"], spec["L"]) == (131, 40, 3) and spec["has_weights"]
    a, b, c = spec["layers"]
    assert (a["mixer"], a["width"], a["blocks"], a["conv"], a["mlp"], a["experts"], a["top"], a["expert_ff"], a["shared_ff"]) == (0, 60, 5, 2, 2, 7, 3, 9, 0)
    assert (b["mixer"], b["heads"], b["kv_heads"], b["dim"], b["vdim"], b["chunk"], b["m_heads"], b["m_dim"], b["m_vdim"], b["mlp"]) == (1, 6, 3, 10, 14, 17, 2, 6, 12, 0)
    assert c["mlp"] == 1 and c["ff"] == 50 and abs(c["left_scale"] - 1.1) < 1e-6 and abs(c["gate_cap"] - 9.0) < 1e-6
    assert abs(spec["logit_scale"] - 0.5) < 1e-7


def test_config_reader_rejects_unknown_layer(kge, tmp_path):
    cfg = oh.make_config()
    cfg["layers"][0]["type"] = "something-else"
    with open(tmp_path / "config.json", "w") as fh:
        json.dump(cfg, fh)
    assert not kge.lib().kge_model_open(str(tmp_path).encode())
    assert b"unknown layer type" in kge.lib().kge_last_error()


def _sched(kge, slots=2, blocks=9, bs=4):
    return kge.lib().kge_sched_create_stateful(8, 64, 64, bs, blocks, 1, -1, slots)


def _add(kge, s, rid, n):
    a = np.arange(n, dtype=np.int32)
    sp = kge.CSamplingParams(4, 0, 1, 0.0, 0, 1.0, 0, None, 0, 0)
    assert kge.lib().kge_sched_add(s, rid, a.ctypes.data, n, C.byref(sp)) == 0


def _run(kge, s, plan):
    ids = np.asarray([p[0] for p in plan], dtype=np.int64)
    cnt = np.asarray([p[1] for p in plan], dtype=np.int32)
    return kge.lib().kge_sched_schedule_scripted(s, ids.ctypes.data, cnt.ctypes.data, len(plan))


def _blocks(kge, s, rid):
    out = np.zeros(64, dtype=np.int32)
    n = kge.lib().kge_sched_request_blocks(s, rid, out.ctypes.data, 64)
    return out[:n].tolist()


def test_scripted_steps_reuse_blocks_and_slots(kge):
    L = kge.lib()
    s = _sched(kge, blocks=7)                   # six usable blocks of four tokens
    _add(kge, s, 1, 10)
    _add(kge, s, 2, 6)
    assert L.kge_sched_state_slot(s, 1) == -1                       # waiting requests hold nothing
    assert _run(kge, s, [(1, 3), (2, 6)]) == 0
    assert {L.kge_sched_state_slot(s, 1), L.kge_sched_state_slot(s, 2)} == {0, 1}
    assert len(_blocks(kge, s, 1)) == 1 and len(_blocks(kge, s, 2)) == 2
    assert _run(kge, s, [(1, 2)]) == 0 and len(_blocks(kge, s, 1)) == 2        # 5 tokens cross a block border
    _add(kge, s, 3, 4)
    assert _run(kge, s, [(3, 4)]) < 0 and b"slot" in L.kge_last_error()       # both slots are taken
    assert L.kge_sched_state_slot(s, 3) == -1 and _blocks(kge, s, 3) == []    # a refused plan changes nothing
    freed_slot, freed_blocks = L.kge_sched_state_slot(s, 2), _blocks(kge, s, 2)
    assert L.kge_sched_abort(s, 2) == 0
    assert _run(kge, s, [(1, 1), (3, 4)]) == 0
    assert L.kge_sched_state_slot(s, 3) == freed_slot                          # the freed slot is used again
    more = np.arange(8, dtype=np.int32)
    assert L.kge_sched_extend(s, 3, more.ctypes.data, 8) == 0
    assert _run(kge, s, [(3, 8)]) == 0
    assert set(freed_blocks) & set(_blocks(kge, s, 3))                         # and so are its blocks
    assert _run(kge, s, [(3, 1)]) < 0 and b"more tokens" in L.kge_last_error()
    assert _run(kge, s, [(1, 4), (1, 1)]) < 0 and b"twice" in L.kge_last_error()
    L.kge_sched_destroy(s)


def test_scripted_steps_refuse_when_blocks_run_out(kge):
    L = kge.lib()
    s = _sched(kge, slots=4, blocks=4)          # three usable blocks of four tokens
    _add(kge, s, 1, 9)
    _add(kge, s, 2, 9)
    assert _run(kge, s, [(1, 8)]) == 0
    assert _run(kge, s, [(2, 8)]) < 0 and b"blocks" in L.kge_last_error()
    assert _run(kge, s, [(2, 4)]) == 0
    n = C.c_int32()
    L.kge_sched_counts(s, None, None, C.byref(n))
    assert n.value == 0
    L.kge_sched_destroy(s)


def test_policy_scheduler_hands_out_slots(kge):
    """The ordinary continuous-batching pass gives every admitted request a slot and takes it back at the end."""
    L = kge.lib()
    s = _sched(kge, slots=2, blocks=33)
    for rid in (1, 2, 3):
        _add(kge, s, rid, 5)
    ids, cnt = np.zeros(8, dtype=np.int64), np.zeros(8, dtype=np.int32)
    assert L.kge_sched_schedule(s, ids.ctypes.data, cnt.ctypes.data, 8) == 2          # the third waits for a slot
    assert sorted(L.kge_sched_state_slot(s, r) for r in (1, 2, 3)) == [-1, 0, 1]
    outs = (kge.StepOutput * 8)()
    toks = np.zeros(2, dtype=np.int32)
    for _ in range(4):                                                                 # max_tokens = 4 ends both
        L.kge_sched_update(s, ids.ctypes.data, toks.ctypes.data, 2, outs, 8)
        k = L.kge_sched_schedule(s, ids.ctypes.data, cnt.ctypes.data, 8)
    assert k == 1 and ids[0] == 3 and L.kge_sched_state_slot(s, 3) in (0, 1)
    L.kge_sched_destroy(s)
