"""Tensor-parallel layers on 2 gloo ranks equal the unsharded fp64 result
(mirrors the scenarios of the reference's test/test_sharding.py and test/test_pp_comm.py)."""
import pytest
import torch

from dist_utils import run_ranks
from xixi_vllm_b200.parallel.pp import PPMissingLayer, divide, get_pp_indices, set_pp_layer_ranges


def _full(shape, seed):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=torch.float64)


def _layers_rank(rank, world):
    from xixi_vllm_b200.models import layers as L
    kw = dict(dtype=torch.float64, device="cpu")
    out = {}
    x = _full((5, 32), 1)
    # column parallel, gathered
    w = _full((48, 32), 2)
    col = L.ColumnParallelLinear(32, 48, gather_output=True, **kw)
    col.load(L.TensorSource({"w": w}), "w")
    out["col"] = (col(x) - x @ w.t()).abs().max().item()
    # row parallel: every rank feeds its slice of the input
    w = _full((24, 32), 3)
    row = L.RowParallelLinear(32, 24, bias=True, **kw)
    b = _full((24,), 4)
    row.load(L.TensorSource({"w": w, "b": b}), "w")
    row.load_bias(L.TensorSource({"b": b}), "b")
    xs = x[:, rank * 16:(rank + 1) * 16]
    out["row"] = (row(xs) - (x @ w.t() + b)).abs().max().item()
    # merged gate|up
    g, u = _full((40, 32), 5), _full((40, 32), 6)
    mg = L.MergedColumnParallelLinear(32, [40, 40], **kw)
    src = L.TensorSource({"g": g, "u": u})
    mg.load(src, "g", 0); mg.load(src, "u", 1)
    y = mg(x)
    ref = torch.cat([(x @ g.t())[:, rank * 20:(rank + 1) * 20], (x @ u.t())[:, rank * 20:(rank + 1) * 20]], -1)
    out["merged"] = (y - ref).abs().max().item()
    # QKV: 4 q heads / 2 kv heads (split) and 4 q heads / 1 kv head (replicated)
    for name, nkv in (("qkv_split", 2), ("qkv_repl", 1)):
        D = 8
        q, k, v = _full((4 * D, 32), 7), _full((nkv * D, 32), 8), _full((nkv * D, 32), 9)
        lay = L.QKVParallelLinear(32, D, 4, nkv, **kw)
        src = L.TensorSource({"q": q, "k": k, "v": v})
        for s in "qkv":
            lay.load(src, s, s)
        kvr = rank if nkv == 2 else 0
        ref = torch.cat([(x @ q.t())[:, rank * 2 * D:(rank + 1) * 2 * D], (x @ k.t())[:, kvr * D:(kvr + 1) * D],
                         (x @ v.t())[:, kvr * D:(kvr + 1) * D]], -1)
        out[name] = (lay(x) - ref).abs().max().item()
        merged = L.QKVParallelLinear(32, D, 4, nkv, **kw)
        merged.load_merged(L.TensorSource({"qkv": torch.cat([q, k, v], 0)}), "qkv")
        out[name + "_merged_load"] = float((merged.weight - lay.weight).abs().max())
    # vocab parallel with padding (vocab 7 pads to 32 over 2 ranks)
    emb_w = _full((7, 6), 10)
    emb = L.VocabParallelEmbedding(7, 6, **kw)
    emb.load(L.TensorSource({"e": emb_w}), "e")
    ids = torch.tensor([0, 6, 3, 3, 5], dtype=torch.int32)
    out["embed"] = (emb(ids) - emb_w[ids.long()]).abs().max().item()
    head = L.ParallelLMHead(7, 6, **kw)
    head.load(L.TensorSource({"e": emb_w}), "e")
    h = _full((5, 6), 11)
    logits = head(h)
    out["head_shape"] = tuple(logits.shape)
    out["head"] = (logits - h @ emb_w.t()).abs().max().item()
    out["argmax"] = bool(torch.equal(head.argmax(h), (h @ emb_w.t()).argmax(-1)))
    return out


def test_parallel_layers_match_unsharded_fp64():
    for res in run_ranks(_layers_rank, world=2, tp=2):
        for k in ("col", "row", "merged", "qkv_split", "qkv_repl", "embed", "head"):
            assert res[k] < 1e-10, (k, res[k])
        assert res["qkv_split_merged_load"] == 0.0 and res["qkv_repl_merged_load"] == 0.0
        assert res["head_shape"] == (5, 7) and res["argmax"]


def _collectives_rank(rank, world):
    from xixi_vllm_b200.parallel import collectives as C
    from xixi_vllm_b200.parallel.groups import get_tp_group
    tp = get_tp_group()
    x = torch.arange(12, dtype=torch.float64).reshape(4, 3) + 100 * rank
    ag0 = C.all_gather(x, tp, dim=0)
    ag1 = C.all_gather(x, tp, dim=-1)
    rs = C.reduce_scatter(torch.ones(4, 3, dtype=torch.float64) * (rank + 1), tp, dim=0)
    ar = C.all_reduce(x.clone(), tp)
    return dict(ag0=tuple(ag0.shape), ag1=tuple(ag1.shape), ag1_ok=bool(torch.equal(ag1[:, 3:], x - 100 * rank + 100)),
                rs=rs.tolist(), ar=float(ar.sum()))


def test_collectives_on_gloo():
    r = run_ranks(_collectives_rank, world=2, tp=2)
    assert r[0]["ag0"] == (8, 3) and r[0]["ag1"] == (4, 6) and r[0]["ag1_ok"]
    assert r[1]["rs"] == [[3.0] * 3] * 2
    assert r[0]["ar"] == r[1]["ar"] == 2 * 66 + 100 * 12


def _pp_rank(rank, world):
    """tp=2 x pp=2: all-reduce inside the TP group, then hidden+residual from stage 0 to stage 1."""
    from xixi_vllm_b200.parallel import collectives as C
    from xixi_vllm_b200.parallel.groups import get_pp_group, get_tp_group
    tp, pp = get_tp_group(), get_pp_group()
    h = torch.full((3, 4), float(rank + 1))
    C.all_reduce(h, tp)
    if pp.is_first_rank:
        for w in C.send_tensors([h, h * 2], group=pp):
            w.wait()
        return None
    a, b = torch.zeros(3, 4), torch.zeros(3, 4)
    C.recv_tensors([a, b], group=pp)
    return (float(a[0, 0]), float(b[0, 0]), tp.ranks, pp.ranks)


def test_pp_handoff_tp2_pp2():
    r = run_ranks(_pp_rank, world=4, tp=2, pp=2)
    assert r[0] is None and r[1] is None
    assert r[2][:2] == (3.0, 6.0) and r[3][:2] == (3.0, 6.0)      # ranks 0+1 summed: 1+2
    assert r[2][2] == [2, 3] and r[2][3] == [0, 2] and r[3][3] == [1, 3]


def _ctrl_rank(rank, world):
    import msgspec

    from xixi_vllm_b200.control.executor import ControlCommand
    from xixi_vllm_b200.data.wire import DecodeBatch, SchedulerOutput
    from xixi_vllm_b200.parallel.control_channel import ControlChannel
    from xixi_vllm_b200.parallel.groups import get_world_group
    ch = ControlChannel(get_world_group().cpu_group)
    enc, dec = msgspec.msgpack.Encoder(), msgspec.msgpack.Decoder(ControlCommand)
    got = []
    for i in range(3):
        cmd = ControlCommand(op="execute", sched=SchedulerOutput(
            decodes=DecodeBatch.of([(i, 9, 5, 1, [4, 5])]), released=[i + 10], step_id=i))
        raw = ch.broadcast(enc.encode(cmd) if rank == 0 else None, src=0)
        c = dec.decode(raw)
        got.append((c.op, c.sched.decodes.bt_vals, c.sched.released, c.sched.step_id))
    if rank == 1:
        ch.send(enc.encode([[1, 2], [3]]), dst=0)
        back = None
    else:
        back = msgspec.msgpack.decode(ch.recv(1))
    last = dec.decode(ch.broadcast(enc.encode(ControlCommand(op="shutdown")) if rank == 0 else None, src=0))
    return got, back, last.op


def test_control_channel_round_trips_schedules():
    r = run_ranks(_ctrl_rank, world=2, tp=2)
    assert r[0][0] == r[1][0] == [("execute", [4, 5], [i + 10], i) for i in range(3)]
    assert r[0][1] == [[1, 2], [3]] and r[0][2] == r[1][2] == "shutdown"


def test_pp_indices_and_helpers():
    assert [get_pp_indices(28, r, 4) for r in range(4)] == [(0, 7), (7, 14), (14, 21), (21, 28)]
    assert [get_pp_indices(10, r, 3) for r in range(3)] == [(0, 3), (3, 6), (6, 10)]     # remainder last
    set_pp_layer_ranges([12, 28])
    try:
        assert [get_pp_indices(40, r, 2) for r in range(2)] == [(0, 12), (12, 40)]
    finally:
        set_pp_layer_ranges(None)
    assert divide(12, 4) == 3
    with pytest.raises(ValueError):
        divide(10, 4)
    x = torch.ones(2)
    assert PPMissingLayer()(x) is x


def _ctl_rank(rank, world, use_shm):
    """Driver broadcasts more messages than the ring has slots, one larger than a slot, then a sentinel."""
    import torch.distributed as dist

    from xixi_vllm_b200.parallel.control_channel import ControlChannel
    from xixi_vllm_b200.parallel.groups import get_world_group
    ch = ControlChannel(get_world_group().cpu_group, shm=use_shm, reply_from=1)
    msgs = [bytes([i % 251]) * (1 + 37 * i) for i in range(40)] + [b"x" * ((1 << 20) + 5), b"", b"end"]
    got = []
    for m in msgs:
        got.append(ch.broadcast(m if rank == 0 else None, src=0))
    # point-to-point replies still work next to the ring
    # replies of the designated rank (ring of its own towards rank 0), small, empty and larger than a slot
    replies = [b"reply", b"", b"y" * ((1 << 20) + 9)] + [bytes([i]) * 100 for i in range(20)]
    if rank == 1:
        for m in replies:
            ch.send(m, dst=0)
    reply = None
    if rank == 0:
        reply = b"reply" if [ch.recv(1) for _ in replies] == replies else b"mismatch"
    # any other pair still talks over gloo
    if rank == 2:
        ch.send(b"side", dst=0)
    if rank == 0:
        assert ch.recv(2) == b"side"
    dist.barrier(group=get_world_group().cpu_group)
    shared = ch.uses_shared_memory
    ch.close()
    return got == msgs, shared, reply


def test_control_channel_ring_and_gloo_paths_deliver_the_same_messages():
    import os

    from dist_utils import run_ranks
    before = {f for f in os.listdir("/dev/shm") if f.startswith("xv_ctl_")} if os.path.isdir("/dev/shm") else set()
    for use_shm in (True, False):
        res = run_ranks(_ctl_rank, world=3, tp=3, args=(use_shm,))
        assert all(ok for ok, _, _ in res)
        assert res[0][2] == b"reply"
        if use_shm and os.path.isdir("/dev/shm"):
            assert all(shared for _, shared, _ in res)
        if not use_shm:
            assert not any(shared for _, shared, _ in res)
    after = {f for f in os.listdir("/dev/shm") if f.startswith("xv_ctl_")} if os.path.isdir("/dev/shm") else set()
    assert after <= before            # the driver removed its ring file
