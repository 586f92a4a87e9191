"""The three calls ferrum-serve's Backend makes of a model (slm_server/src/backend.rs:72-155) on
token ids, with the cross-request batching the reference's model thread does not have (it scores
requests one by one, slm_server/src/model_thread.rs:29-38). Text, tokenizer, HTTP and JSON stay
with the caller: this is the seam a `Backend::Cuda` variant calls through.

A CudaBackend owns one model on one GPU and is used from one thread (the model thread). Scoring
requests queued with `submit_score` / `submit_score_rolling` are answered together by `flush()`:
their windows share forward passes (fc_score_requests). Generation is served one request at a
time (`generate`), as the reference serves it.
"""
from dataclasses import dataclass, field

import numpy as np

from . import engine


@dataclass
class GenRequest:
    """The numeric fields of backend.rs GenRequest."""
    prompt: list
    max_tokens: int = 64
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    repetition_penalty: float = 1.0
    seed: int = 0
    eos: int = -1
    cancel: object = None      # numpy int32[1] flag the connection handler sets, or None


@dataclass
class _Pending:
    ids: np.ndarray
    start: int
    ticket: int
    rolling: bool = False


@dataclass
class CudaBackend:
    model: engine.CudaSlm
    batch_windows: int = 32
    _queue: list = field(default_factory=list)
    _tickets: int = 0

    # ---- /v1/loglikelihood and /v1/loglikelihood_rolling ---------------------------------
    def submit_score(self, context_ids, continuation_ids):
        """GenerativeSLM::score (slm/scoring.rs:95-131): the continuation given the context."""
        ctx, cont = list(context_ids), list(continuation_ids)
        if not ctx:
            raise engine.FerrumCudaError(engine._lib.FC_E_DIM, "score: the context must hold at least one token (pass BOS)")
        return self._push(np.asarray(ctx + cont, dtype=np.int32), len(ctx), False)

    def submit_score_rolling(self, ids):
        """GenerativeSLM::score_rolling (slm/scoring.rs:136-140): every token but the first."""
        return self._push(np.asarray(list(ids), dtype=np.int32), 1, True)

    def _push(self, ids, start, rolling):
        self._tickets += 1
        self._queue.append(_Pending(ids, start, self._tickets, rolling))
        return self._tickets

    def flush(self):
        """Answers every queued scoring request: {ticket: reply dict as backend.rs builds it}."""
        pending, self._queue = self._queue, []
        if not pending:
            return {}
        scores = self.model.score_requests([(p.ids, p.start) for p in pending], self.batch_windows)
        out = {}
        for p, s in zip(pending, scores):
            out[p.ticket] = ({"logprob": s.logprob, "n_tokens": s.n_tokens} if p.rolling
                             else {"logprob": s.logprob, "n_tokens": s.n_tokens, "greedy": s.greedy})
        return out

    def score(self, context_ids, continuation_ids):
        t = self.submit_score(context_ids, continuation_ids)
        return self.flush()[t]

    def score_rolling(self, ids):
        t = self.submit_score_rolling(ids)
        return self.flush()[t]

    # ---- /v1/generate ---------------------------------------------------------------------
    def generate(self, g):
        """backend.rs:107-155: None for a request whose client already left, else the new ids."""
        if g.cancel is not None and int(g.cancel[0]):
            return None
        if g.temperature <= 0.0 and g.repetition_penalty == 1.0:
            toks, _ = self.model.generate_tokens(g.prompt, g.max_tokens, eos=g.eos, cancel=g.cancel)
        else:
            params = engine.sampling(g.temperature, g.top_k, g.top_p, g.repetition_penalty)
            toks, _ = self.model.generate_sampled(g.prompt, g.max_tokens, params, rng_state=engine._lib.lib().fc_rng_seed(g.seed),
                                                  eos=g.eos, cancel=g.cancel)
        return {"tokens": [int(t) for t in toks], "n_tokens": int(len(toks))}
