"""Transfer-side admission and request lifecycle of a stage: the hooks the PD connector calls on its engine.

The reference spreads these over ``StageEngine`` and ``Scheduler``
(vllm_rlt/engine/stage_engine.py:679-775, vllm_rlt/core/scheduler.py:347-447). A PD handoff needs exactly this
much of them, and nothing of the compute scheduling around it:

* ``reserve_transfer``: create the stage-local request of one transfer generation, look the prompt up in the
  decode side's prefix cache, budget the reservation against what the requests already admitted may still
  grow by, allocate the whole prompt's pages (reusing cached prefix pages) and pin them with a transfer lease.
  A reservation that does not fit leaves nothing behind and may be retried.
* ``accept_import``: after every remote write has landed, publish the imported range, offer the prompt's
  pages to the prefix cache and queue the request for a compute slot.
* ``release_transfer_compute`` / ``release_transfer`` / ``suspend_transfer``: retire the source side in two
  steps (compute state when the last staging read is done, KV when remote access has provably ended) and
  park a cancelled export.

``TransferStage`` has the attributes ``PDStageConnector`` reads from a stage engine (``cache_manager``,
``scheduler.requests``, ``scheduler.config``, ``stage_config``, ``model.config.hidden_size``), so the connector
runs against it unchanged. In a deployment whose engine is the reference's ``StageEngine`` the connector
talks to that instead, with the same results (pinned by traces recorded from it).
"""

from __future__ import annotations

import enum
from dataclasses import dataclass, field, replace
from types import SimpleNamespace

from .kv_pool import KVPool


class Phase(enum.Enum):
    """Where a transferred request stands on this stage (names of vllm_rlt/request.py's RequestPhase)."""

    WAITING = "waiting"            # outgoing: competes for a prefill slot; incoming: imported, waits for a compute slot
    RECEIVING = "receiving"        # incoming: pages reserved, remote writes may be in flight
    PREFILL = "prefill"            # outgoing: prompt being computed
    TRANSFERRING = "transferring"  # outgoing: compute finished or cancelled, KV still leased to the transfer
    DECODE = "decode"              # incoming: admitted to compute
    FINISHED = "finished"


@dataclass
class StageRequest:
    """The stage-local face of one transfer generation (the fields of ``Request`` the handoff touches)."""

    request_id: str
    prompt_token_ids: list
    sampling_params: object
    phase: Phase
    trace_id: str | None = None
    num_prefilled_tokens: int = 0
    hidden_state: object = None
    compute_released: bool = False

    @property
    def max_tokens(self) -> int:
        return int(self.sampling_params.max_tokens)


@dataclass(frozen=True)
class AdmissionPlan:
    """What admitting one request would take; a description, not a reservation
    (vllm_rlt/core/scheduler.py:110-129). All block counts are over all planes."""

    capacity_tokens: int        # logical capacity: prompt + outputs - 1 (the last sampled token is never fed back)
    initial_tokens: int         # tokens whose pages are taken now
    prefix_blocks: tuple        # cached pages reused, one tuple of per-plane blocks each
    cached_tokens: int
    required_blocks: int        # fresh blocks this admission is charged for
    reserved_growth_blocks: int  # blocks promised to requests admitted earlier
    admission_headroom_blocks: int
    cached_claim_blocks: int    # reused blocks that so far counted as free (held by the cache alone)

    @property
    def total_budget_blocks(self) -> int:
        return (self.required_blocks + self.reserved_growth_blocks + self.admission_headroom_blocks
                + self.cached_claim_blocks)


@dataclass
class StageSettings:
    max_num_seqs: int = 8
    prefill_chunk_size: int = 2048
    enable_preemption: bool = False
    wavefront_chunked_prefill: bool = False


class TransferStage:
    def __init__(self, role: str, pool: KVPool, *, settings: StageSettings | None = None, hidden_size: int = 16,
                 stage_id: str | None = None):
        if role not in ("prefill", "decode", "prefill_decode"):
            raise ValueError("role must be prefill, decode or prefill_decode")
        self.cache_manager = pool
        self.settings = settings or StageSettings()
        self.requests: dict[str, StageRequest] = {}
        self.waiting: list[str] = []  # imports accepted and waiting for a compute slot, oldest first
        # the attribute paths the connector uses on a stage engine
        self.scheduler = SimpleNamespace(requests=self.requests, config=self.settings)
        self.stage_config = SimpleNamespace(role=role, produces_tokens=role != "prefill", accepts_prompt=role != "decode",
                                            stage_id=stage_id or f"{role}-0")
        self.model = SimpleNamespace(config=SimpleNamespace(hidden_size=hidden_size))

    # ------------------------------------------------------------------ admission

    def reserved_growth_blocks(self, *, reserve_outputs: bool) -> int:
        """Blocks that look free but are promised to the growth of requests already here
        (vllm_rlt/core/scheduler.py:347-374): a prompt in prefill will need its remaining pages; without
        preemption every request that owns pages will also need room for its outputs."""
        pool = self.cache_manager
        promised = 0
        for request in self.requests.values():
            owns = pool.has_allocation(request.request_id)
            if request.phase is not Phase.PREFILL and not (reserve_outputs and owns):
                continue
            tokens = len(request.prompt_token_ids)
            if reserve_outputs:
                tokens += request.max_tokens - 1
            promised += max(0, pool.required_blocks(tokens) - pool.allocated_blocks(request.request_id))
        return promised

    def plan_admission(self, request: StageRequest, active: int) -> AdmissionPlan:
        """Prefix reuse, pages taken now and the budget charged (vllm_rlt/core/scheduler.py:376-420).
        The lookup refreshes the cache's recency order, so this is not a pure read."""
        pool = self.cache_manager
        prompt = len(request.prompt_token_ids)
        capacity = prompt + request.max_tokens - 1
        prefix = pool.lookup_prefix(request.prompt_token_ids)
        cached = len(prefix) * pool.block_size
        incremental = pool.incremental_allocation
        initial = min(prompt, cached + self.settings.prefill_chunk_size) if incremental else capacity
        reserve_outputs = incremental and not self.settings.enable_preemption
        budget_tokens = prompt if incremental and not reserve_outputs else capacity
        return AdmissionPlan(
            capacity_tokens=capacity,
            initial_tokens=initial,
            prefix_blocks=prefix,
            cached_tokens=cached,
            required_blocks=pool.required_blocks(budget_tokens) - len(prefix) * pool.storage_depths,
            reserved_growth_blocks=self.reserved_growth_blocks(reserve_outputs=reserve_outputs),
            admission_headroom_blocks=pool.watermark_blocks if active else 0,
            cached_claim_blocks=pool.exclusive_prefix_blocks(prefix),
        )

    def reserve_transfer(self, request_id, prompt_token_ids, sampling_params, *, receiving, trace_id=None):
        """One stage-local request per transfer generation, its whole prompt mapped and leased
        (vllm_rlt/engine/stage_engine.py:679-710, vllm_rlt/core/scheduler.py:422-447). ``None``: admission failed
        and neither a request nor an allocation was kept. On success ``request.num_prefilled_tokens`` is the
        decode side's prefix hit, which the connector reports as ``cached_tokens`` with the tables."""
        if request_id in self.requests:
            raise ValueError(f"request {request_id!r} already exists")
        tokens = list(prompt_token_ids)
        if not tokens:
            raise ValueError("prompt must not be empty")
        request = StageRequest(request_id, tokens, sampling_params, Phase.WAITING, trace_id)
        pool = self.cache_manager
        occupied = any(pool.has_allocation(rid) for rid in self.requests)
        plan = self.plan_admission(request, int(occupied))
        if pool.incremental_allocation:
            plan = replace(plan, initial_tokens=len(tokens))  # a transfer needs the whole prompt mapped up front
        if plan.total_budget_blocks > pool.num_free_blocks or not pool.allocate(
                request_id, plan.capacity_tokens, initial_tokens=plan.initial_tokens, prefix=plan.prefix_blocks):
            return None
        pool.pin_transfer(request_id, request_id)
        self.requests[request_id] = request
        request.num_prefilled_tokens = plan.cached_tokens
        if receiving:
            request.phase = Phase.RECEIVING
        return request

    # ------------------------------------------------------------------ import activation

    def accept_import(self, request: StageRequest, hidden, *, cached_tokens: int = 0) -> bool:
        """Every remote write of this generation has landed: publish the KV and queue the request for compute
        (vllm_rlt/engine/stage_engine.py:751-775). False for a stale generation (the id was reused)."""
        if self.requests.get(request.request_id) is not request:
            return False
        if request.phase is not Phase.RECEIVING or request.request_id in self.waiting:
            raise ValueError("request is not awaiting an import")
        count = len(request.prompt_token_ids)
        pool = self.cache_manager
        pool.mark_imported_prefix(request.request_id, count, start=cached_tokens)
        pool.publish_prefix(request.request_id, request.prompt_token_ids, count)
        request.num_prefilled_tokens = count
        request.hidden_state = hidden
        self.waiting.append(request.request_id)  # stays RECEIVING, and leased, until a compute slot is granted
        return True

    def grant_compute(self, limit: int | None = None) -> list[StageRequest]:
        """The scheduler's part: give waiting imports a compute slot, oldest first, up to ``max_num_seqs``
        running at once. The transfer lease ends here; the allocation is the request's own from now on."""
        running = sum(r.phase is Phase.DECODE for r in self.requests.values())
        granted = []
        while self.waiting and running < self.settings.max_num_seqs and (limit is None or len(granted) < limit):
            request = self.requests[self.waiting.pop(0)]
            request.phase = Phase.DECODE
            self.cache_manager.unpin_transfer(request.request_id, request.request_id)
            running += 1
            granted.append(request)
        return granted

    def finish(self, request: StageRequest) -> None:
        """A decode request produced its last token: drop it and its KV."""
        if self.requests.get(request.request_id) is request:
            del self.requests[request.request_id]
            request.phase = Phase.FINISHED
            self.cache_manager.free(request.request_id)

    # ------------------------------------------------------------------ source retirement

    def begin_prefill(self, request: StageRequest) -> None:
        request.phase = Phase.PREFILL

    def end_prefill(self, request: StageRequest, hidden) -> None:
        """The prompt is computed: the request now only waits for its transfer to drain."""
        request.num_prefilled_tokens = len(request.prompt_token_ids)
        request.hidden_state = hidden
        request.phase = Phase.TRANSFERRING

    def suspend_transfer(self, request: StageRequest):
        """Cancel future computation of an export; in-flight state and the lease stay
        (vllm_rlt/engine/stage_engine.py:712-714)."""
        if self.requests.get(request.request_id) is request:
            request.phase = Phase.TRANSFERRING

    def release_transfer_compute(self, request: StageRequest, *, ready_event) -> bool:
        """Drop compute state once the connector's last staging read is done; KV and the staging row stay leased
        (vllm_rlt/engine/stage_engine.py:716-731). Non-blocking; a stale request releases nothing."""
        if self.requests.get(request.request_id) is not request:
            return False
        if request.phase is not Phase.TRANSFERRING:
            raise ValueError("request is not awaiting transfer completion")
        if not ready_event.query():
            return False
        request.hidden_state = None
        request.compute_released = True
        return True

    def release_transfer(self, request: StageRequest) -> bool:
        """Remote access to this generation's KV has ended: forget the request, drop the lease, free the pages
        (vllm_rlt/engine/stage_engine.py:733-749)."""
        if self.requests.get(request.request_id) is not request:
            return False
        rid = request.request_id
        del self.requests[rid]
        if rid in self.waiting:
            self.waiting.remove(rid)
        request.phase = Phase.FINISHED
        pool = self.cache_manager
        if pool.has_allocation(rid):
            pool.free(rid)  # deferred by the lease ...
        if pool.has_allocation(rid):
            pool.unpin_transfer(rid, rid)  # ... and carried out when it is dropped
        return True
