"""Case matrix runner: every case is one ``bench.py`` invocation in its own process (tree), with a per-case time
limit; a case that fails or runs out of time is recorded with ``ok: false`` and the matrix goes on
(reference: bench/run_matrix.py:116-149, bench/cases.py).

    python -m bench.matrix --suite smoke            # one GPU, a minute or two
    python -m bench.matrix --suite tp               # Qwen3-8B at TP = 1 .. visible GPUs, both arms
    python -m bench.matrix --suite decode --only tp2
    python -m bench.matrix --suite full --out bench/out/matrix.jsonl

Each result line is the JSON line bench.py printed plus ``case``, ``ok``, ``seconds`` and, on failure, the end of
the case's output. ``python -m bench.report <file>`` renders the file as a table.
"""

from __future__ import annotations

import argparse
import json
import os
import signal
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def visible_gpus() -> int:
    try:
        import torch

        return int(torch.cuda.device_count())
    except Exception:  # noqa: BLE001
        return 0


def _case(tag, gpus=1, impl="ours", limit=600, **flags):
    return dict(tag=tag, gpus=gpus, impl=impl, limit=limit, flags=flags)


def suites(n_gpus: int) -> dict:
    tps = [n for n in (1, 2, 4, 8) if n <= max(1, n_gpus)]
    s = {
        "smoke": [_case("0.6b-steady", model="Qwen3-0.6B", steps=16, warmup=3, max_num_seqs=64, limit=240),
                  _case("0.6b-decode32", model="Qwen3-0.6B", mode="decode", decode_batch=32, steps=32, limit=240)],
        "tp": [_case(f"8b-tp{n}-{impl}", gpus=n, impl=impl, steps=64, warmup=6)
               for n in tps for impl in ("reference", "ours")],
        "decode": [_case(f"8b-tp{n}-decode{b}-{impl}", gpus=n, impl=impl, mode="decode", decode_batch=b, steps=64)
                   for n in tps for b in (1, 32, 256) for impl in ("reference", "ours")],
        "full": [_case(f"8b-tp{n}-512req-{impl}", gpus=n, impl=impl, mode="full", requests=512, limit=1200)
                 for n in tps for impl in ("reference", "ours")],
        "pp": [_case(f"8b-tp{max(1, n // 2)}pp2-mb{m}", gpus=n, pp=2, pp_microbatches=m, steps=48)
               for n in tps if n >= 2 for m in (1, 2)],
    }
    if n_gpus >= 8:
        s["32b"] = [_case(f"32b-tp8-{impl}", gpus=8, impl=impl, mode="full", model="Qwen3-32B", requests=256,
                          prompt_min=4096, prompt_max=4096, out_tokens=1024, limit=1500)
                    for impl in ("reference", "ours")]
        s["32b"].append(_case("32b-tp4pp2", gpus=8, pp=2, mode="full", model="Qwen3-32B", requests=256,
                              prompt_min=4096, prompt_max=4096, out_tokens=1024, limit=1500))
    return s


def command(case: dict, port: int) -> list[str]:
    flags = []
    for k, v in case["flags"].items():
        flags += [f"--{k.replace('_', '-')}", str(v)]
    base = ["bench.py", "--gpus", str(case["gpus"]), "--impl", case["impl"], *flags]
    if case["gpus"] > 1:
        return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(case["gpus"]),
                "--master-addr", "127.0.0.1", "--master-port", str(port), *base]
    return [sys.executable, *base]


def run_case(case: dict, port: int) -> dict:
    t0 = time.time()
    p = subprocess.Popen(command(case, port), cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                         start_new_session=True)
    try:
        out, _ = p.communicate(timeout=case["limit"])
        timed_out = False
    except subprocess.TimeoutExpired:
        timed_out = True
        os.killpg(p.pid, signal.SIGTERM)             # the process group this runner started
        try:
            out, _ = p.communicate(timeout=20)
        except subprocess.TimeoutExpired:
            os.killpg(p.pid, signal.SIGKILL)
            out, _ = p.communicate()
    rec = {}
    for line in (out or "").splitlines():
        if line.startswith("{"):
            try:
                rec = json.loads(line)
            except ValueError:
                pass
    ok = (not timed_out) and p.returncode == 0 and "value" in rec
    rec.update(case=case["tag"], ok=ok, seconds=round(time.time() - t0, 1))
    if not ok:
        rec["error"] = ("time limit" if timed_out else f"exit {p.returncode}") + ": " + (out or "")[-400:]
    return rec


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--suite", default="smoke")
    ap.add_argument("--only", default="", help="run the cases whose tag contains this")
    ap.add_argument("--out", default=os.path.join(ROOT, "bench", "out", "matrix.jsonl"))
    ap.add_argument("--list", action="store_true")
    a = ap.parse_args()
    table = suites(visible_gpus())
    if a.suite not in table:
        raise SystemExit(f"unknown suite {a.suite!r}; have {sorted(table)}")
    cases = [c for c in table[a.suite] if a.only in c["tag"]]
    if a.list:
        for c in cases:
            print(c["tag"], " ".join(command(c, 29900)))
        return
    os.makedirs(os.path.dirname(a.out), exist_ok=True)
    port = 29900
    with open(a.out, "a") as f:
        for c in cases:
            port += 16
            rec = run_case(c, port)
            f.write(json.dumps(rec) + "\n")
            f.flush()
            print(f"{c['tag']:32s} ok={rec['ok']} {rec.get('value', '')} {rec.get('unit', '')} ({rec['seconds']} s)", flush=True)


if __name__ == "__main__":
    main()
