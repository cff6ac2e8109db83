"""Public facade (reference: src/control/engine.py:29-294).

Owns the tokenizer, validates and truncates requests, mirrors request state for streaming,
and drives an ``EngineCoreClient``. It does not know how TP/PP/DP are laid out.
"""

from __future__ import annotations

import warnings
from collections.abc import Iterator
from dataclasses import replace

from ..config import EngineConfig
from ..data import Sequence, SequenceStatus
from ..sampling_params import SamplingParams
from ..utils.tokenizer import load_tokenizer
from .client import InprocClient, make_client

__all__ = ["Engine"]


class Engine:
    """``add_request`` / ``step`` for continuous batching, ``generate_batch`` for blocking
    batches, ``generate`` for token streaming."""

    def __init__(self, config: EngineConfig, executor=None) -> None:
        import torch

        self.config = config
        if config.device == "cpu":
            self.device = torch.device("cpu")
        else:
            first = config.device_ids[0] if config.device_ids else 0
            self.device = torch.device(f"cuda:{first}")
        self.dtype = resolve_dtype(config)
        self.tokenizer = load_tokenizer(config.model, config.hf_config.vocab_size)
        eos = getattr(self.tokenizer, "eos_token_id", None)
        if eos is None:
            eos = config.hf_config.get("eos_token_id", 0)
        if isinstance(eos, (list, tuple)):
            eos = eos[0]
        self.eos_token_id = int(eos if eos is not None else 0)
        self.context_len = config.context_len
        self.block_size = config.block_size
        self._client = make_client(config, eos_token_id=self.eos_token_id, device=self.device,
                                   dtype=self.dtype, executor=executor)
        # dp=1: the very objects the scheduler mutates. dp>1: mirrors advanced from step outputs.
        self._seqs: dict[int, Sequence] = {}

    # --- introspection ------------------------------------------------------------------
    def _core(self):
        if not isinstance(self._client, InprocClient):
            raise NotImplementedError("only reachable for the in-process (dp=1) engine")
        return self._client.engine_core

    @property
    def scheduler(self):
        return self._core().scheduler

    @property
    def metrics(self):
        return self._core().metrics

    @property
    def last_num_cached_tokens(self) -> int:
        if not isinstance(self._client, InprocClient):
            return 0
        return self._client.engine_core.last_num_cached_tokens

    def reset_kv(self, prefix_backend: str | None = None) -> None:
        """Drop all cached KV and rebuild the scheduler, optionally switching prefix backend."""
        if not isinstance(self._client, InprocClient):
            raise NotImplementedError("reset_kv is only supported for dp=1")
        if prefix_backend is not None and prefix_backend not in ("none", "hash", "radix"):
            raise ValueError(f"invalid prefix_backend: {prefix_backend!r}")
        self._client.engine_core.reset_kv(prefix_backend)

    # --- requests ----------------------------------------------------------------------
    def add_request(self, prompt: str | list[int], sampling_params: SamplingParams | None = None) -> Sequence:
        sp = sampling_params or SamplingParams()
        ids = list(prompt) if isinstance(prompt, (list, tuple)) else self.tokenizer.encode(prompt)
        if not ids:
            raise ValueError("empty prompt")
        if len(ids) > self.context_len:
            warnings.warn(
                f"prompt length {len(ids)} > context_len={self.context_len}; "
                f"truncating to last {self.context_len} tokens", stacklevel=2)
            ids = ids[-self.context_len:]
        room = max(0, self.context_len - len(ids))
        if sp.max_tokens > room:
            warnings.warn(
                f"max_tokens={sp.max_tokens} + prompt={len(ids)} exceeds context_len="
                f"{self.context_len}; clamping max_tokens to {room}", stacklevel=2)
            sp = replace(sp, max_tokens=room)
        seq = Sequence.from_prompt(ids, block_size=self.block_size, sampling=sp)
        self._seqs[seq.seq_id] = seq
        self._client.add_request(seq)
        return seq

    def step(self) -> tuple[list[tuple[int, list[int]]], int]:
        """One schedule -> forward -> sample -> update round.

        Returns (finished, metric): ``finished`` lists ``(seq_id, completion_token_ids)`` of
        requests that ended this step; ``metric`` is the number of tokens processed.
        """
        outputs, metric = self._client.step()
        mirror = not isinstance(self._client, InprocClient)
        finished: list[tuple[int, list[int]]] = []
        if not mirror:
            # in-process core: the Sequence objects are shared and already up to date; only ends matter
            for out in outputs:
                if out.is_finished:
                    seq = self._seqs.pop(out.seq_id, None)
                    if seq is not None:
                        finished.append((out.seq_id, seq.token_ids[seq.num_prompt_tokens:]))
            return finished, metric
        for out in outputs:
            seq = self._seqs.get(out.seq_id)
            if seq is None:
                continue
            if mirror:
                for tid in out.new_token_ids:
                    seq.append_token(tid)
                if out.is_finished:
                    seq.status = SequenceStatus.FINISHED
            if out.is_finished:
                finished.append((out.seq_id, seq.token_ids[seq.num_prompt_tokens:]))
                del self._seqs[out.seq_id]
        return finished, metric

    def generate_batch(self, prompts, sampling_params=None) -> list[str]:
        """Blocking generation; results come back in input order."""
        sps = self._broadcast_params(prompts, sampling_params)
        seqs = [self.add_request(p, sp) for p, sp in zip(prompts, sps)]
        texts: dict[int, str] = {}
        while self.has_unfinished():
            for seq_id, completion in self.step()[0]:
                texts[seq_id] = self.tokenizer.decode(completion)
        return [texts[s.seq_id] for s in seqs]

    def generate(self, prompt, max_new_tokens: int = 128, temperature: float = 0.0,
                 top_p: float | None = None, top_k: int | None = None,
                 min_p: float | None = None) -> Iterator[str]:
        """Streams one decoded string per generated token."""
        sp = SamplingParams(temperature=temperature, top_p=top_p, top_k=top_k, min_p=min_p,
                            max_tokens=max_new_tokens)
        seq = self.add_request(prompt, sp)
        sent = 0
        while not seq.is_finished:
            self.step()
            while sent < seq.num_known_completion_tokens:     # tokens still in flight on the device are not shown
                yield self.tokenizer.decode([seq.token_ids[seq.num_prompt_tokens + sent]])
                sent += 1

    def has_unfinished(self) -> bool:
        return self._client.has_unfinished()

    @staticmethod
    def _broadcast_params(prompts, sampling_params) -> list[SamplingParams]:
        if sampling_params is None:
            return [SamplingParams() for _ in prompts]
        if isinstance(sampling_params, SamplingParams):
            return [sampling_params] * len(prompts)
        if len(sampling_params) != len(prompts):
            raise ValueError("sampling_params length must match prompts")
        return list(sampling_params)

    def destroy(self) -> None:
        self._client.destroy()
        self._seqs.clear()


def resolve_dtype(config: EngineConfig):
    """``dtype="auto"`` follows the checkpoint's ``torch_dtype``; bf16 if it names none."""
    import torch

    name = config.dtype
    if name == "auto":
        name = config.hf_config.get("torch_dtype") or "bfloat16"
    if not isinstance(name, str):
        return name
    name = name.replace("torch.", "")
    dtype = {"float16": torch.float16, "half": torch.float16, "bfloat16": torch.bfloat16,
             "float32": torch.float32, "float": torch.float32, "float64": torch.float64}[name]
    if dtype != torch.bfloat16 and getattr(config, "device", "cuda") == "cuda":
        # The reference serves whatever the checkpoint declares and falls back to float16
        # (reference: src/control/engine.py:79-84); the sm_100a kernels here are bf16 only.
        raise ValueError(f"dtype {name} is not supported on CUDA: the sm_100a kernels of this engine run bfloat16 "
                         f"activations and weights only. Pass dtype=\"bfloat16\" (a float16 / float32 checkpoint is "
                         f"converted while it is loaded) or run on device=\"cpu\".")
    return dtype
