"""Batch staging, sampler oracle, graph buckets, CLI plumbing (CPU)."""
import sys
from unittest import mock

import numpy as np
import pytest
import torch

from xixi_vllm_b200.data.wire import DecodeBatch, SchedulerOutput, SeqSchedule
from xixi_vllm_b200.ops import cpu_ref
from xixi_vllm_b200.runtime.graphs import make_bs_list
from xixi_vllm_b200.runtime.staging import BatchStager


def test_stager_packs_decodes_then_prefills_and_tracks_table_tails():
    st = BatchStager(max_seqs=8, max_tokens=128, max_blocks=8, block_size=16, device="cpu")
    pre = SeqSchedule(seq_id=1, num_cached_tokens=0, token_ids=list(range(100, 120)), bt_from=0, bt_tail=[3, 5],
                      need_sample=True, temperature=0.7, top_k=5)
    b = st.build(SchedulerOutput(prefills=[pre]))
    assert b.num_tokens == 20 and b.n_prefill == 1 and not b.all_greedy
    assert b.positions.tolist() == list(range(20))
    assert b.slots.tolist() == [3 * 16 + i for i in range(16)] + [5 * 16 + i for i in range(4)]
    assert b.attn.cu_q.tolist() == [0, 20] and b.attn.kv_lens.tolist() == [20]
    assert b.sample_rows.tolist() == [19] and b.top_k.tolist() == [5]
    # next step: decode of seq 1 (no new pages on the wire) + chunk of a new seq 2 with a cached prefix
    dec = DecodeBatch.of([(1, 7, 20, 2, [])])
    pre2 = SeqSchedule(seq_id=2, num_cached_tokens=16, token_ids=[1, 2, 3], bt_from=0, bt_tail=[6, 2],
                       need_sample=False)
    b = st.build(SchedulerOutput(decodes=dec, prefills=[pre2]))
    assert b.input_ids.tolist() == [7, 1, 2, 3] and b.positions.tolist() == [20, 16, 17, 18]
    assert b.slots.tolist() == [5 * 16 + 4, 2 * 16, 2 * 16 + 1, 2 * 16 + 2]
    assert b.attn.num_decode == 1 and b.attn.kv_lens.tolist() == [21, 19] and b.attn.cu_q.tolist() == [0, 1, 4]
    assert b.attn.block_tables[0, :2].tolist() == [3, 5] and b.attn.block_tables[1, :2].tolist() == [6, 2]
    assert b.sample_rows.tolist() == [0] and b.prefill_sampled == [False] and not b.all_greedy
    assert abs(b.temperature.tolist()[0] - 0.7) < 1e-6 and b.top_k.tolist() == [5]    # remembered from the prefill
    # page growth arrives as a tail; release drops the row
    b = st.build(SchedulerOutput(decodes=DecodeBatch.of([(1, 9, 32, 2, [4])]), released=[2]))
    assert b.slots.tolist() == [4 * 16] and 2 not in st.row_of
    # padding to a graph bucket adds inert rows
    b = st.build(SchedulerOutput(decodes=DecodeBatch.of([(1, 9, 33, 3, [])])), pad_to=4, fixed_blocks=True)
    assert b.num_tokens == 4 and b.slots.tolist()[1:] == [-1, -1, -1] and b.attn.kv_lens.tolist() == [34, 0, 0, 0]
    assert b.attn.block_tables.shape == (4, 8) and b.num_samples == 4


def test_stager_python_and_native_fill_agree():
    rng = np.random.default_rng(0)
    outs = []
    for use_native in (True, False):
        st = BatchStager(max_seqs=16, max_tokens=64, max_blocks=16, block_size=16, device="cpu")
        if not use_native:
            st._lib = None
        rng = np.random.default_rng(0)
        entries = []
        for i in range(10):
            cached = int(rng.integers(0, 200))
            nb = cached // 16 + 1
            entries.append((i + 1, int(rng.integers(1000)), cached, 0, rng.integers(0, 99, size=nb).tolist()))
        b = st.build(SchedulerOutput(decodes=DecodeBatch.of(entries)))
        outs.append((b.positions.tolist(), b.slots.tolist(), b.attn.kv_lens.tolist(), b.attn.block_tables.tolist()))
    assert outs[0] == outs[1]


def test_filtered_probs_rules():
    logits = torch.tensor([[4.0, 3.0, 2.0, 1.0, 0.0]])
    one = torch.tensor([1.0])
    p = cpu_ref.filtered_probs(logits, one, torch.tensor([2]), one, torch.tensor([0.0]))[0]
    assert (p > 0).tolist() == [True, True, False, False, False] and abs(float(p.sum()) - 1) < 1e-6
    full = torch.softmax(logits[0], -1)
    p = cpu_ref.filtered_probs(logits, one, torch.tensor([0]), torch.tensor([0.7]), torch.tensor([0.0]))[0]
    # 0.64 of the mass precedes token 1 (<= 0.7, kept), 0.87 precedes token 2 (dropped)
    assert (p > 0).tolist() == [True, True, False, False, False]
    p = cpu_ref.filtered_probs(logits, one, torch.tensor([0]), one, torch.tensor([0.2]))[0]
    assert (p > 0).tolist() == (full >= 0.2 * full[0]).tolist()
    g = torch.Generator().manual_seed(0)
    ids = cpu_ref.sample(logits.expand(2000, 5), torch.ones(2000), torch.full((2000,), 2), torch.ones(2000),
                         torch.zeros(2000), g)
    assert set(ids.tolist()) == {0, 1}
    assert cpu_ref.sample(logits, torch.tensor([0.0]), torch.tensor([0]), one, torch.tensor([0.0])).tolist() == [0]


def test_graph_buckets():
    assert make_bs_list(1) == [1]
    assert make_bs_list(8) == [1, 2, 4, 8]
    bl = make_bs_list(256)
    assert bl[:5] == [1, 2, 4, 8, 16] and bl[-1] == 256 and 128 in bl and 160 in bl and 144 not in bl
    assert make_bs_list(100)[-1] == 100


def test_cli_precedence_and_cleanup(tmp_path):
    """YAML overrides defaults, flags override YAML; destroy() runs exactly once on every exit path
    (mirrors the reference's test/test_entrypoint_cleanup.py with a mocked engine)."""
    root = __import__("os").path.dirname(__import__("os").path.dirname(__import__("os").path.abspath(__file__)))
    sys.path.insert(0, root)
    import run
    y = tmp_path / "c.yaml"
    y.write_text("max_new_tokens: 7\ntp_size: 2\nprefix_backend: radix\nunknown_key: 1\n")
    args = run.build_parser().parse_args(["--config", str(y), "--tp", "4", "--cg", "--prefix-backend", "none",
                                          "--device-ids", "3,2,1,0", "--pp-layer-counts", "12,28"])
    cfg = run.config_from_args(args)
    assert cfg["max_new_tokens"] == 7 and cfg["tp_size"] == 4 and cfg["prefix_backend"] == "none"
    assert cfg["enforce_eager"] is False and cfg["device_ids"] == [3, 2, 1, 0] and cfg["pp_layer_counts"] == [12, 28]
    assert "unknown_key" not in cfg and cfg["kvcache_block_size"] == 16

    for fail_at in (None, "warmup", "generate"):
        engine = mock.Mock()
        engine.tokenizer.encode.return_value = [1, 2, 3]
        engine.tokenizer.decode.return_value = "x"
        seq = mock.Mock(is_finished=True, num_completion_tokens=1, token_ids=[1, 2, 3, 4], num_prompt_tokens=3)
        engine.add_request.return_value = seq
        if fail_at == "generate":
            engine.add_request.side_effect = RuntimeError("boom")
        warm = mock.Mock(return_value=0.0, side_effect=RuntimeError("warm") if fail_at == "warmup" else None)
        with mock.patch.object(run, "_make_engine", return_value=engine), mock.patch.object(run, "_warmup", warm), \
                mock.patch.object(run, "cuda_sync"):
            for fn in (run.run_single, run.run_batch):
                engine.destroy.reset_mock()
                if fail_at:
                    with pytest.raises(RuntimeError):
                        fn(dict(cfg, prompt="hi", temperature=0.0, top_p=None, top_k=None))
                else:
                    fn(dict(cfg, prompt="hi", temperature=0.0, top_p=None, top_k=None))
                assert engine.destroy.call_count == 1


def test_split_forward_batch_pieces_cover_the_batch_in_order():
    """Micro-batches for pipeline stages: whole sequences, rebased offsets, samples in the original order."""
    import numpy as np
    from xixi_vllm_b200.data import KVManager, Sequence
    from xixi_vllm_b200.control.scheduler import Scheduler
    from xixi_vllm_b200.runtime.staging import split_forward_batch
    from xixi_vllm_b200.sampling_params import SamplingParams
    kv = KVManager(num_blocks=64, block_size=16, prefix_backend="none")
    sch = Scheduler(kv, max_num_seqs=8, max_num_batched_tokens=40, eos_token_id=1)
    for n in (5, 9, 30, 40):
        sch.add(Sequence.from_prompt(list(range(3, 3 + n)), block_size=16,
                                     sampling=SamplingParams(max_tokens=4, ignore_eos=True)))
    st = BatchStager(max_seqs=8, max_tokens=128, max_blocks=8, block_size=16, device="cpu")
    seen_partial = False
    for _ in range(4):                       # prefill-only step, then mixed steps with a mid-prompt chunk
        b = sch.schedule()
        full = st.build(b.to_wire())
        for parts in (1, 2, 3, 16):
            pieces = split_forward_batch(full, parts)
            assert len(pieces) <= max(1, min(parts, full.attn.num_seqs))
            assert pieces[0][1] == 0 and pieces[-1][2] == full.num_tokens
            rows, samples, seqs = [], [], 0
            for sub, t0, t1 in pieces:
                assert t1 - t0 == sub.num_tokens == int(sub.attn.cu_q[-1]) and int(sub.attn.cu_q[0]) == 0
                assert torch.equal(sub.input_ids, full.input_ids[t0:t1])
                assert sub.attn.num_seqs == sub.attn.kv_lens.numel() == sub.attn.block_tables.shape[0]
                assert sub.n_decode + sub.n_prefill == sub.attn.num_seqs and sub.attn.num_decode == sub.n_decode
                assert sub.attn.max_q_len == int(np.diff(sub.attn.cu_q_host).max())
                assert len(sub.prefill_sampled) == sub.n_prefill and sub.num_samples == sub.sample_rows.numel()
                rows.append(sub.sample_rows + t0)
                samples.append(sub.temperature)
                seqs += sub.attn.num_seqs
            assert seqs == full.attn.num_seqs
            assert torch.equal(torch.cat(rows), full.sample_rows)
            assert torch.cat(samples).numel() == full.num_samples
        seen_partial |= not all(full.prefill_sampled)
        sch.update(b, [7] * len(b.prefills), [7] * len(b.decodes))
    assert seen_partial


def test_token_references_into_the_previous_steps_samples():
    """One-step-late scheduling: a decode row whose input token the host did not know yet carries -(row) - 1,
    the index of its sample in the previous step; the stager flags such batches and the ids are patched from
    that step's sample buffer before the forward."""
    from xixi_vllm_b200.ops import dispatch as ops
    st = BatchStager(max_seqs=8, max_tokens=64, max_blocks=4, block_size=16, device="cpu")
    pre = [SeqSchedule(seq_id=i, num_cached_tokens=0, token_ids=[10 + i, 20 + i], bt_from=0, bt_tail=[i],
                       need_sample=True) for i in (1, 2, 3)]
    b = st.build(SchedulerOutput(prefills=pre))
    assert b.num_token_refs == 0
    prev = torch.tensor([501, 502, 503], dtype=torch.int64)           # samples of that step, in row order
    # next step: sequences 3 and 1 refer to rows 2 and 0, sequence 2's token is already known
    dec = DecodeBatch.of([(3, -3, 2, 1, []), (2, 77, 2, 1, []), (1, -1, 2, 1, [])])
    b = st.build(SchedulerOutput(decodes=dec))
    assert b.num_token_refs == 3 and b.input_ids.tolist() == [-3, 77, -1]
    ops.resolve_token_refs(b.input_ids[: b.num_token_refs], prev)
    assert b.input_ids.tolist() == [503, 77, 501]
    b = st.build(SchedulerOutput(decodes=DecodeBatch.of([(3, 5, 3, 1, []), (2, 6, 3, 1, [])])))
    assert b.num_token_refs == 0


def test_bench_matrix_records_failures_and_time_limits(monkeypatch):
    """The case runner keeps going: a case that exits non-zero, prints no result line or runs out of time is
    recorded with ok=false (and its process group is ended), a good case carries bench.py's JSON line."""
    from bench import matrix

    scripts = {
        "good": 'import json; print("noise"); print(json.dumps({"value": 12.5, "unit": "tokens/s"}))',
        "crash": 'import sys; print("boom"); sys.exit(3)',
        "silent": 'print("no json here")',
        "hang": 'import time; print("started", flush=True); time.sleep(60)',
    }
    monkeypatch.setattr(matrix, "command", lambda case, port: [sys.executable, "-c", scripts[case["tag"]]])
    good = matrix.run_case(dict(tag="good", gpus=1, impl="ours", limit=30, flags={}), 0)
    assert good["ok"] and good["value"] == 12.5 and good["case"] == "good"
    crash = matrix.run_case(dict(tag="crash", gpus=1, impl="ours", limit=30, flags={}), 0)
    assert not crash["ok"] and crash["error"].startswith("exit 3") and "boom" in crash["error"]
    silent = matrix.run_case(dict(tag="silent", gpus=1, impl="ours", limit=30, flags={}), 0)
    assert not silent["ok"]
    hang = matrix.run_case(dict(tag="hang", gpus=1, impl="ours", limit=1, flags={}), 0)
    assert not hang["ok"] and hang["error"].startswith("time limit") and hang["seconds"] < 30
    # the command line of a multi-GPU case goes through torch.distributed.run on 127.0.0.1
    monkeypatch.undo()
    cmd = matrix.command(dict(tag="t", gpus=4, impl="reference", limit=1, flags={"decode_batch": 32, "mode": "decode"}), 29950)
    assert "--nproc-per-node" in cmd and "127.0.0.1" in cmd and cmd[-4:] == ["--decode-batch", "32", "--mode", "decode"]
    assert any(c["gpus"] == 8 for c in matrix.suites(8)["32b"]) and "32b" not in matrix.suites(2)
