"""Data parallelism: ``dp_size`` independent engine replicas in child processes, reached
over ZMQ ``ipc://`` PUSH/PULL pairs (reference: src/control/mp_client.py:34-294).

Each replica owns a scheduler, a KV ledger and a ``tp*pp`` rank world on its own slice of
the devices. Requests go round-robin by arrival; ``step`` blocks until at least one replica
reports and then drains whatever else is ready. Differences from the reference: replicas
start concurrently, the readiness timeout scales with model size instead of a fixed 60 s,
and a replica that dies is detected (its pending requests are reported as failed) instead
of blocking the facade forever.
"""

from __future__ import annotations

import copy
import multiprocessing as mp
import shutil
import tempfile
import time

import msgspec
import zmq

from ..config import EngineConfig
from ..data import EngineCoreOutput, Sequence
from .client import EngineCoreClient

__all__ = ["MPClient", "RequestWire", "CoreRequest", "CoreOutput", "run_engine_core_proc"]


class RequestWire(msgspec.Struct):
    seq_id: int
    token_ids: list[int]
    block_size: int
    temperature: float
    top_p: float | None
    top_k: int | None
    min_p: float | None
    max_tokens: int
    ignore_eos: bool

    @classmethod
    def from_sequence(cls, s: Sequence) -> "RequestWire":
        return cls(s.seq_id, list(s.token_ids), s.block_size, s.temperature, s.top_p, s.top_k,
                   s.min_p, s.max_tokens, s.ignore_eos)

    def to_sequence(self) -> Sequence:
        return Sequence(token_ids=list(self.token_ids), block_size=self.block_size, seq_id=self.seq_id,
                        num_prompt_tokens=len(self.token_ids), last_token=self.token_ids[-1],
                        temperature=self.temperature, top_p=self.top_p, top_k=self.top_k,
                        min_p=self.min_p, max_tokens=self.max_tokens, ignore_eos=self.ignore_eos)


class CoreRequest(msgspec.Struct):
    op: str                       # "add" | "shutdown"
    req: RequestWire | None = None


class CoreOutput(msgspec.Struct):
    outputs: list[EngineCoreOutput]
    metric: int = 0
    error: str | None = None


def run_engine_core_proc(config: EngineConfig, *, eos_token_id: int, device: str, dtype, in_addr: str,
                         out_addr: str, ready) -> None:
    """Replica main loop: drain requests, step while there is work, push each step's outputs."""
    from .core import EngineCore

    assert config.dp_size == 1, "replica config must have dp_size 1"
    ctx = zmq.Context()
    in_sock = ctx.socket(zmq.PULL)
    in_sock.bind(in_addr)
    out_sock = ctx.socket(zmq.PUSH)
    out_sock.bind(out_addr)
    enc = msgspec.msgpack.Encoder()
    dec = msgspec.msgpack.Decoder(CoreRequest)
    core = None
    try:
        core = EngineCore(config, eos_token_id=eos_token_id, device=device, dtype=dtype)
        ready.set()
        while True:
            stop = False
            # block briefly when idle instead of spinning
            timeout = 0 if core.has_unfinished() else 5
            while in_sock.poll(timeout):
                timeout = 0
                msg = dec.decode(in_sock.recv())
                if msg.op == "shutdown":
                    stop = True
                    break
                if msg.op == "add" and msg.req is not None:
                    core.add_request(msg.req.to_sequence())
            if stop:
                break
            if core.has_unfinished():
                try:
                    outputs, metric = core.step()
                except Exception as e:  # report, then die: the facade fails the pending requests
                    out_sock.send(enc.encode(CoreOutput(outputs=[], error=f"{type(e).__name__}: {e}")))
                    raise
                if outputs or metric:
                    out_sock.send(enc.encode(CoreOutput(outputs=outputs, metric=metric)))
    finally:
        if core is not None:
            core.destroy()
        in_sock.close(0)
        out_sock.close(1000)
        ctx.term()


class MPClient(EngineCoreClient):
    def __init__(self, config: EngineConfig, *, eos_token_id: int, device=None, dtype=None) -> None:
        assert config.dp_size > 1
        self.config, self.dp_size = config, config.dp_size
        self._ctx = zmq.Context()
        self._enc = msgspec.msgpack.Encoder()
        self._dec = msgspec.msgpack.Decoder(CoreOutput)
        self._in: list = []
        self._out: list = []
        self._sock_replica: dict = {}
        self._poller = zmq.Poller()
        self._procs: list = []
        self._pending: dict[int, int] = {}     # seq_id -> replica
        self._next = 0
        self._tmp = tempfile.mkdtemp(prefix="xv_dp_")
        ctx = mp.get_context("spawn")
        events = []
        try:
            for r in range(self.dp_size):
                rc = self._replica_config(r)
                in_addr, out_addr = f"ipc://{self._tmp}/in_{r}", f"ipc://{self._tmp}/out_{r}"
                ev = ctx.Event()
                dev = f"cuda:{rc.device_ids[0]}" if rc.device == "cuda" else "cpu"
                p = ctx.Process(target=run_engine_core_proc, args=(rc,), daemon=False,
                                kwargs=dict(eos_token_id=eos_token_id, device=dev, dtype=dtype,
                                            in_addr=in_addr, out_addr=out_addr, ready=ev))
                p.start()
                self._procs.append(p)
                events.append(ev)
                s_in = self._ctx.socket(zmq.PUSH)
                s_in.connect(in_addr)
                s_out = self._ctx.socket(zmq.PULL)
                s_out.connect(out_addr)
                self._in.append(s_in)
                self._out.append(s_out)
                self._sock_replica[s_out] = r
                self._poller.register(s_out, zmq.POLLIN)
            deadline = time.monotonic() + self._ready_timeout()
            for r, ev in enumerate(events):
                while not ev.wait(timeout=0.2):
                    if not self._procs[r].is_alive():
                        raise RuntimeError(f"DP replica {r} exited with code {self._procs[r].exitcode} during start-up")
                    if time.monotonic() > deadline:
                        raise RuntimeError(f"DP replica {r} failed to initialize in time")
        except BaseException:
            self.destroy()
            raise

    def _ready_timeout(self) -> float:
        if self.config.dp_ready_timeout_s > 0:
            return self.config.dp_ready_timeout_s
        c = self.config.hf_config
        params = c.num_hidden_layers * (4 * c.hidden_size * c.hidden_size + 3 * c.hidden_size * c.intermediate_size)
        return 120.0 + params / 1e9 * 30.0     # ~30 s per billion parameters on top of a base

    def _replica_config(self, r: int) -> EngineConfig:
        """Replica r: dp=1, its own ``tp*pp`` device slice, rendezvous port offset by 16*r."""
        per = self.config.tp_size * self.config.pp_size
        if self.config.device_ids is not None:
            devices = self.config.device_ids[r * per:(r + 1) * per]
            if len(devices) != per:
                raise ValueError(f"device_ids length {len(self.config.device_ids)} incompatible with "
                                 f"dp={self.dp_size} x (tp*pp={per})")
        else:
            devices = list(range(r * per, (r + 1) * per))
        rc = copy.copy(self.config)
        rc.dp_size = 1
        rc.device_ids = devices
        rc.nccl_port = self.config.nccl_port + 16 * r
        rc.seed = self.config.seed + r
        return rc

    def add_request(self, seq: Sequence) -> None:
        r = self._next
        self._next = (self._next + 1) % self.dp_size
        self._pending[seq.seq_id] = r
        self._in[r].send(self._enc.encode(CoreRequest(op="add", req=RequestWire.from_sequence(seq))))

    def step(self):
        return self._drain(block=True)

    def has_unfinished(self) -> bool:
        return bool(self._pending)

    def _fail_replica(self, r: int, why: str) -> list[EngineCoreOutput]:
        lost = [sid for sid, rr in self._pending.items() if rr == r]
        for sid in lost:
            del self._pending[sid]
        if lost:
            raise RuntimeError(f"DP replica {r} failed ({why}); lost requests: {sorted(lost)}")
        return []

    def _drain(self, *, block: bool):
        outputs: list[EngineCoreOutput] = []
        metric = 0
        got_any = False
        while True:
            if block and not got_any:
                ready = dict(self._poller.poll(200))
                if not ready:
                    for r, p in enumerate(self._procs):
                        if not p.is_alive() and any(rr == r for rr in self._pending.values()):
                            self._fail_replica(r, f"process exited with code {p.exitcode}")
                    if not self._pending:
                        break
                    continue
            else:
                ready = dict(self._poller.poll(0))
                if not ready:
                    break
            for sock in ready:
                msg = self._dec.decode(sock.recv())
                if msg.error is not None:
                    self._fail_replica(self._sock_replica[sock], msg.error)
                outputs.extend(msg.outputs)
                metric += msg.metric
                for o in msg.outputs:
                    if o.is_finished:
                        self._pending.pop(o.seq_id, None)
            got_any = True
        return outputs, metric

    def destroy(self) -> None:
        for s in self._in:
            try:
                s.send(self._enc.encode(CoreRequest(op="shutdown")), zmq.NOBLOCK)
            except zmq.ZMQError:
                pass
        for p in self._procs:
            p.join(timeout=15)
            if p.is_alive():
                p.terminate()
                p.join(timeout=5)
        for s in self._in + self._out:
            s.close(0)
        self._ctx.term()
        self._procs.clear()
        self._pending.clear()
        shutil.rmtree(self._tmp, ignore_errors=True)
