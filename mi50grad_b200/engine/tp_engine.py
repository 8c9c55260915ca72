"""Tensor-parallel engine: one process per GPU, ranks joined by
`torch.distributed`, collectives issued from inside this package's kernels over
NVLink symmetric memory.

API-compatible with the reference's `TPInferenceEngine` (reference:
src/inference/tp_engine.py:1718-6843), which is ONE process driving every GPU
with `hipSetDevice` switching, host-recorded events between GPUs and ten
interchangeable dispatch modes (reference: src/inference/tp_engine.py:2753-2800).
Here every rank constructs the same object and calls the same methods in the
same order; the per-token step is a single CUDA graph per rank and GPUs
synchronise through flags in peer memory, so the dispatch-mode toggles of the
reference survive only as no-op shims that record what was asked for.
"""
from __future__ import annotations

import logging
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch
import torch.distributed as dist

from ..config import AR_MODES, EngineConfig, QwenConfig
from ..models.weights import LayerWeights, ModelWeights
from ..parallel.sharding import make_shard_spec, shard_layer
from .engine import InferenceEngine

log = logging.getLogger(__name__)


class TPInferenceEngine:
    def __init__(self, config: QwenConfig, device_ids: Optional[Sequence[int]] = None,
                 max_seq_len: int = 2048, quant_format: str = "w4a16", use_int4_attention: bool = False,
                 engine_config: Optional[EngineConfig] = None, max_batch: int = 1):
        self.config = config
        if dist.is_available() and dist.is_initialized():
            self.tp_size, self.tp_rank = dist.get_world_size(), dist.get_rank()
        else:
            self.tp_size, self.tp_rank = 1, 0
        if device_ids is not None and len(device_ids) != self.tp_size:
            raise ValueError(f"{len(device_ids)} device ids but {self.tp_size} ranks: launch one process "
                             "per GPU (torch.distributed.run) and initialise the process group first")
        self.device_ids = list(device_ids) if device_ids is not None else list(range(self.tp_size))
        self.ecfg = (engine_config or EngineConfig()).replace(tp_size=self.tp_size, tp_rank=self.tp_rank)
        device_id = torch.cuda.current_device()
        self.comm = None
        if self.tp_size > 1:
            from ..parallel.symm import SymmComm
            self.comm = SymmComm(hidden=config.hidden_size, part_floats=min(512, max_seq_len) * config.hidden_size,
                                 use_multimem=self.ecfg.use_multimem, wait_us=self.ecfg.wait_budget_us)
        self.engine = InferenceEngine(config, device_id, max_seq_len, self.tp_size, self.tp_rank, quant_format,
                                      use_int4_attention, self.ecfg, self.comm, max_batch)
        self.engines = [self.engine]          # reference attribute name; one entry: this rank
        self.spec = make_shard_spec(config, self.tp_size, self.tp_rank)
        self._requested: Dict[str, object] = {}
        self._spec_mode = None

    # ------------------------------------------------------------------ weights
    def load_layer_weights(self, layer_idx: int, weights, sharded: bool = False):
        """`weights`: full (unsharded) engine-format layer; this rank keeps its shard
        (reference: src/inference/tp_engine.py:1887-1890)."""
        if isinstance(weights, dict):
            weights = LayerWeights(**weights)
        lw = weights if sharded or self.tp_size == 1 else shard_layer(weights, self.config, self.tp_size, self.tp_rank)
        self.engine.load_layer_weights(layer_idx, lw)

    def load_final_norm(self, weight):
        self.engine.load_final_norm(torch.as_tensor(weight))

    def load_lm_head(self, weight, sharded: bool = False):
        w = torch.as_tensor(weight)
        if not sharded and self.tp_size > 1:
            a, b = self.spec.vocab
            w = w[a:b]
        self.engine.load_lm_head(w)

    def load_embedding(self, weight):
        self.engine.load_embedding(torch.as_tensor(weight))

    def load_model(self, mw: ModelWeights, sharded: bool = False):
        for i, lw in enumerate(mw.layers):
            self.load_layer_weights(i, lw, sharded)
        self.load_embedding(mw.embed)
        self.load_lm_head(mw.lm_head, sharded)
        self.load_final_norm(mw.final_norm)

    def init_random(self, seed: int = 0, int4_attention: bool = True):
        self.engine.init_random(seed, int4_attention)

    # ------------------------------------------------------------------ stepping
    def reset(self, seq: Optional[int] = None):
        self.engine.states.reset(seq)

    def prefill_tokens(self, tokens, seq: int = 0) -> int:
        return self.engine.prefill_tokens(tokens, seq)

    def decode_tokens(self, n_steps: int, seqs=None, graph=None, collect: bool = True):
        self._before_step()
        out = self.engine.decode_tokens(n_steps, seqs, graph, collect)
        self._after_step()
        return out

    def step_tokens(self, tokens, seq: int = 0, logits: bool = True, commit: bool = True):
        self._before_step()
        out = self.engine.step_tokens(tokens, seq, logits, commit)
        self._after_step()
        return out

    def score_tokens(self, tokens, seq: int = 0):
        return self.engine.score_tokens(tokens, seq)

    def perplexity(self, tokens, seq: int = 0) -> float:
        return self.engine.perplexity(tokens, seq)

    def generate_tokens(self, prompt, n_new: int, seq: int = 0, graph=None):
        self._before_step()
        out = self.engine.generate_tokens(prompt, n_new, seq, graph)
        self._after_step()
        return out

    def step_host(self, token: int, seq: int = 0) -> int:
        self._before_step()
        out = self.engine.step_host(token, seq)
        self._after_step()
        return out

    def prefill_step(self, token_embeddings, seq: int = 0):
        return self.engine.prefill_step(token_embeddings, seq)

    def decode_step(self, token_embedding, position: Optional[int] = None, seq: int = 0):
        return self.engine.decode_step(token_embedding, position, seq)

    def decode_step_batch(self, token_embeddings: List, positions: List[int], seq: int = 0) -> List:
        """Several tokens of ONE sequence at contiguous positions in one step (a
        draft-verification step), like the reference's TP batch decode (reference:
        src/inference/tp_engine.py:2856-2862).  Multi-sequence decode is
        `decode_tokens(seqs=[...])`."""
        if positions and positions[0] != self.engine.states.length(seq):
            self.engine.states.set_length(seq, positions[0])
        embs = torch.stack([torch.as_tensor(e).float() for e in token_embeddings])
        out = self.engine.forward_embeddings(embs, seq)
        if isinstance(token_embeddings[0], np.ndarray):
            return [o.cpu().numpy() for o in out]
        return [o.clone() for o in out]

    # ------------------------------------------------------------------ speculation
    def spec_step(self, drafts, parents, seqs=None, roots=None):
        """One-pass verify-and-commit for several sequences (engine.InferenceEngine.spec_step)."""
        self._before_step()
        out = self.engine.spec_step(drafts, parents, seqs, roots)
        self._after_step()
        return out

    def spec_step_tokens(self, root: int, drafts, parents, seq: int = 0):
        return self.engine.spec_step_tokens(root, drafts, parents, seq)

    def decode_step_tree(self, token_embeddings: List, tree_mask, kv_embeddings=None, seq: int = 0) -> List:
        """Hidden states of every node of a draft tree from ONE forward pass, nothing
        committed (reference: src/inference/tp_engine.py:3070-3341).  `tree_mask` is a
        generate.tree_attention.TreeAttentionMask (its topology gives the parents) or a
        list of parent indices.  Unlike the reference, nodes get RoPE position
        length + depth, draft K/V go to scratch slots beyond the committed length, and
        the DeltaNet layers follow the tree.  `kv_embeddings` is not needed: the
        committed KV cache is used."""
        topo = getattr(tree_mask, "tree", None) or getattr(tree_mask, "topology", None)
        parents = list(topo.parents()) if topo is not None else [int(p) for p in tree_mask]
        embs = torch.stack([torch.as_tensor(e).float() for e in token_embeddings])
        out = self.engine.forward_embeddings_tree(embs, parents, seq)
        if isinstance(token_embeddings[0], np.ndarray):
            return [o.cpu().numpy() for o in out]
        return [o.clone() for o in out]

    def set_speculative_mode(self, enabled: bool, ngram_size: int = 3, max_draft_len: int = 5):
        """(reference: src/inference/tp_engine.py:6597-6631)  Buffers for verification are
        always allocated; this records the draft parameters used by generate.speculative."""
        self._spec_mode = {"ngram_size": ngram_size, "max_draft_len": max_draft_len} if enabled else None
        self.ecfg = self.ecfg.replace(spec_ngram=ngram_size, spec_max_draft=max_draft_len)

    def decode_step_speculative(self, token_embeddings: List, position: int, draft_tokens: List[int], seq: int = 0):
        """Hidden state after each of the given embeddings (pending token first, then
        the drafts) from one pass, nothing committed; returns (hidden states, number of
        drafts) like the reference (src/inference/tp_engine.py:6633-6678).  The caller
        compares lm_head(hidden[i]) with draft i+1; `spec_step` does all of it on the
        device and is what the generators use."""
        if position != self.engine.states.length(seq):
            self.engine.states.set_length(seq, position)
        n = len(token_embeddings)
        hs = self.decode_step_tree(token_embeddings, list(range(-1, n - 1)), seq=seq)
        return hs, len(draft_tokens)

    def set_eagle_mode(self, enabled: bool, k_draft: int = 5, temperature: float = 0.0):
        """(reference: src/inference/tp_engine.py:6680-6708)"""
        self._eagle = {"k_draft": k_draft, "temperature": temperature} if enabled else None

    def generate_eagle_drafts(self, hidden_state, k: Optional[int] = None) -> List[int]:
        """k draft tokens from a final-normed hidden state with the model's own head:
        token = argmax(lm_head(h)), h <- normalised embedding of the token (reference:
        src/inference/tp_engine.py:6710-6794, which zeroes the hidden state after the
        first token).  Logits come from the device lm_head, all ranks get the same ids."""
        k = k if k is not None else (getattr(self, "_eagle", None) or {}).get("k_draft", 5)
        eng = self.engine
        eng._ensure_driver()
        from ..ops import kernels as K
        from ..ops import lib as L
        # the whole loop stays on the device: lm_head GEMV on this rank's vocabulary slice, arg-max across
        # the ranks inside the arg-max kernel (symmetric memory), embedding gather + norm; one host read at the end
        h16 = torch.as_tensor(hidden_state).float().flatten().to(eng.device).half().reshape(1, -1)
        toks = torch.empty(k, dtype=torch.int32, device=eng.device)
        ctx = eng._comm_ctx() if self.tp_size > 1 else None
        for i in range(k):
            K.gemv(eng.lm_head, h16, out=eng.buf["logits"][:1], mode=L.EPI_STORE_F32,
                   scratch=eng.buf["gemv_scratch"], counters=eng.buf["gemv_counters"])
            tok = K.argmax(eng.buf["logits"][:1, :eng.spec.vocab_local], eng.spec.vocab[0], eng.argmax_blocks, ctx)
            toks[i:i + 1] = tok[:1]
            e = eng.embed.index_select(0, tok[:1].long()).float()
            h16 = (e * torch.rsqrt(e.pow(2).mean(-1, keepdim=True) + self.config.rms_norm_eps)).half()
        return toks.tolist()

    def decode_step_eagle(self, hidden_state, position: int, seq: int = 0):
        """Draft with `generate_eagle_drafts`, verify and commit in one pass; returns
        (accepted draft tokens, next pending token).  The pending token is the one the
        last step stored for the sequence."""
        if position != self.engine.states.length(seq):
            self.engine.states.set_length(seq, position)
        k = (getattr(self, "_eagle", None) or {}).get("k_draft", 5)
        drafts = self.generate_eagle_drafts(hidden_state, k + 1)[1:]
        return self.engine.spec_step([drafts], [list(range(-1, len(drafts) - 1))], [seq])[0]

    def compute_logits(self, hidden=None):
        """fp32 logits over the full vocabulary on every rank (the slices are
        all-gathered; the reference computes logits on GPU 0 only:
        src/inference/tp_engine.py:2529-2530)."""
        local = self.engine.compute_logits(hidden)
        if self.tp_size == 1:
            return local
        t = torch.as_tensor(local).to(self.engine.device)
        vl = -(-self.config.vocab_size // self.tp_size)
        pad = torch.zeros(vl, device=t.device)
        pad[:t.numel()] = t
        outs = [torch.empty_like(pad) for _ in range(self.tp_size)]
        dist.all_gather(outs, pad)
        full = torch.cat(outs)[:self.config.vocab_size]
        return full.cpu().numpy() if isinstance(local, np.ndarray) else full

    def synchronize(self):
        self.engine.synchronize()

    def check_status(self):
        """Raise CommTimeout if a bounded device wait expired since the last check; with failure detection
        on, the expiry is also published so that the peers stop before their next step."""
        if self.comm is None:
            return
        try:
            self.comm.check_status()
        except Exception as e:
            hb = getattr(self, "_heartbeat", None)
            if hb is not None:
                hb.mark_failed(str(e)[:200])
            raise

    # ------------------------------------------------------------------ failure detection / recovery
    def enable_failure_detection(self, store=None, heartbeat_s: float = 0.2, timeout_s: float = 5.0):
        """Start a heartbeat for this rank and check the peers' before every step: a rank that exited,
        hung on the host or reported a device-wait expiry makes the others raise `RankFailure` at their
        next step boundary instead of entering an exchange that cannot complete (the kernels' bounded
        waits cover the case where the peer dies inside a step).  `store`: any object with set/get
        (default: the torch.distributed store of the bootstrap)."""
        from ..utils.watchdog import DictStore, Heartbeat, Watchdog
        if store is None:
            if dist.is_available() and dist.is_initialized():
                store = dist.distributed_c10d._get_default_store()
            else:
                store = DictStore()
        self._heartbeat = Heartbeat(store, self.tp_rank, interval_s=heartbeat_s).start()
        self._watchdog = Watchdog(store, self.tp_rank, self.tp_size, timeout_s=timeout_s)
        return self

    def disable_failure_detection(self):
        hb = getattr(self, "_heartbeat", None)
        if hb is not None:
            hb.stop()
        self._heartbeat = self._watchdog = None

    def _before_step(self):
        wd = getattr(self, "_watchdog", None)
        if wd is not None:
            wd.check(require_present=False)

    def _after_step(self):
        hb = getattr(self, "_heartbeat", None)
        if hb is not None:
            hb.beat(self.engine._steps)

    def snapshot_all(self, seqs=None):
        """Snapshots of the given sequence slots (default: all), for `recover`."""
        seqs = range(self.engine.max_batch) if seqs is None else seqs
        return [self.engine.states.snapshot(s) for s in seqs]

    def recover(self, snapshots=(), group=None):
        """After a failed exchange (CommTimeout / RankFailure) on a process group that is whole again
        (the failed rank was restarted, or the ranks re-initialised torch.distributed): throw the old
        symmetric-memory communicator away, rendezvous a new one on `group` (default: the world), rebuild
        the step driver on it and put every snapshotted sequence back.  Collective: every rank calls it.
        The world size must be the one the weights were sharded for."""
        from ..parallel.symm import SymmComm
        if self.tp_size > 1:
            world = dist.get_world_size(group) if group is not None else dist.get_world_size()
            if world != self.tp_size:
                raise ValueError(f"recover() on {world} ranks, but the weights are sharded for {self.tp_size}")
            old = self.comm
            self.comm = SymmComm(hidden=self.config.hidden_size,
                                 part_floats=old.part_floats if old is not None else None,
                                 use_multimem=self.ecfg.use_multimem, wait_us=self.ecfg.wait_budget_us, group=group)
            if old is not None:
                old.close()
            self.engine.comm = self.comm
        self.engine._drop_driver()
        self.engine._graph_key = None
        for s in snapshots:
            self.engine.states.restore(s)
        hb = getattr(self, "_heartbeat", None)
        if hb is not None:
            hb.clear_failed()
            hb.beat(self.engine._steps)
        if self.tp_size > 1:
            dist.barrier(group)               # every rank has withdrawn its mark before anyone checks again
        return self.comm

    def launches_per_step(self) -> int:
        return self.engine.launches_per_step()

    def streamed_bytes_per_token(self) -> int:
        return self.engine.streamed_bytes_per_token()

    def build_dispatch_cache(self):
        self.engine.build_decode_launch_cache()

    def cleanup(self):
        self.disable_failure_detection()
        self.engine.cleanup()
        if self.comm is not None:
            self.comm.close()

    # ------------------------------------------------------------------ counters
    def get_allreduce_call_count(self) -> int:
        """All-reduces issued so far: every exchange fused into a projection or collective kernel, as
        counted by the step driver while it issues and replays steps."""
        return self.engine.exchange_count() - getattr(self, "_ar_base", 0)

    def reset_allreduce_counter(self):
        self._ar_base = 0
        self._ar_base = self.get_allreduce_call_count()

    # ------------------------------------------------------------------ reference toggles
    def _note(self, name, value):
        self._requested[name] = value

    def set_deferred_attention_ar(self, enabled: bool, consistent: bool = False):
        """Deferred attention all-reduce (reference: src/inference/tp_engine.py:2368-2409).
        `consistent=True` selects the variant whose residual streams re-converge."""
        mode = ("deferred_consistent" if consistent else "deferred_ref") if enabled else "exact"
        self.set_ar_mode(mode)

    def set_ar_mode(self, mode: str):
        if mode not in AR_MODES:
            raise ValueError(mode)
        self.ecfg = self.ecfg.replace(ar_mode=mode)
        self.engine.ecfg = self.engine.ecfg.replace(ar_mode=mode)
        self.engine._drop_driver()

    def set_graph_dispatch(self, enabled: bool):
        self.ecfg = self.ecfg.replace(use_graph=bool(enabled))
        self.engine.ecfg = self.engine.ecfg.replace(use_graph=bool(enabled))

    set_global_graph_dispatch = set_graph_dispatch

    def set_c_dispatch(self, enabled: bool):
        """The C++ step driver is the only dispatch path; kept for API parity."""
        self._note("c_dispatch", enabled)

    def set_c_dispatch_v2(self, enabled: bool): self._note("c_dispatch_v2", enabled)
    def set_cached_dispatch(self, enabled: bool): self._note("cached_dispatch", enabled)
    def set_stream_overlap_dispatch(self, enabled: bool): self._note("stream_overlap", enabled)
    def set_threaded_dispatch(self, enabled: bool): self._note("threaded", enabled)
    def set_persistent_kernel(self, enabled: bool):
        """Persistent decode dispatch (reference: src/inference/tp_engine.py set_persistent_kernel,
        src/kernels/persistent_decode.hip:271-468, a stub there).  Here: the projection-chain kernel
        (csrc/chain.cu) runs the consecutive INT4 projections of the decode step as one resident launch
        each (`EngineConfig.use_chain = 1`); disabling returns to the default for the rank count."""
        self._note("persistent_kernel", enabled)
        want = 1 if enabled else -1
        if int(self.engine.ecfg.use_chain) != want:
            self.engine.ecfg = self.engine.ecfg.replace(use_chain=want)
            self.ecfg = self.ecfg.replace(use_chain=want)
            self.engine._drop_driver()
    def set_direct_kv_write(self, enabled: bool): self._note("direct_kv_write", enabled)
    def set_awq_mode(self, enabled: bool = True): self._note("awq", enabled)
    def set_kernel_p2p_allreduce(self, enabled: bool): self._note("kernel_p2p", enabled)
    def set_fused_p2p_reduce(self, enabled: bool): self._note("fused_p2p", enabled)
    def set_ring_allreduce(self, enabled: bool): self._note("ring", enabled)
    def set_batched_allreduce_enabled(self, enabled: bool): self._note("batched_ar", enabled)
    def set_double_buffer_enabled(self, enabled: bool): self._note("double_buffer", enabled)
    def set_weight_prefetch(self, enabled: bool): self._note("weight_prefetch", enabled)

    def set_compressed_allreduce(self, enabled: bool):
        """INT8-compressed all-reduce was rejected by the reference's own data
        (cosine 0.87) and NVLink makes it pointless; refused explicitly."""
        if enabled:
            raise NotImplementedError("compressed all-reduce is not provided")

    def requested_toggles(self) -> Dict[str, object]:
        return dict(self._requested)
