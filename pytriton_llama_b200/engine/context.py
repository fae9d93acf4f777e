"""What one step looks like to the parts: the flat batch on the device and the cache views.

A step carries ``T`` tokens of ``R`` requests, request after request.  Nothing in here says
whether a request is in its prompt or decoding: a portion is ``q_len`` new tokens that follow
``ctx_len - q_len`` tokens already in the cache.  (lite_llama hands its layers an ``AttentionInfo``
with the cache buffers, ``cur_select_index`` and ``b_req_tokens_table`` for the same purpose,
lite_llama/executor/executor_struct.py:13-23, and tells prompt from decode by the sequence length,
lite_llama/models/llama.py:62-118.)
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import torch


@dataclass
class GroupStepView:
    """Paging data of one cache group for this step."""
    page_size: int
    block_table: torch.Tensor   # int32 [R, max_pages]; -1 where a page was given back or never held
    slots: torch.Tensor         # int32 [T]; page * page_size + offset of each new token, -1 = do not store
    window: int = 0


@dataclass
class LayerCacheView:
    """The cache entry one run of a layer uses."""
    group: Optional[GroupStepView]
    kv: Optional[torch.Tensor]      # [pages, 2, kv_heads, page_size, head_dim] of this entry; with values of another
                                    # size [pages, kv_heads * page_size * (head_dim + value_dim)], keys first
    state: Optional[torch.Tensor]   # [slots, *state_shape] per-request state of this entry
    write: bool = True              # False: read what another run of a layer stored
    states: Dict[str, torch.Tensor] = field(default_factory=dict)   # named per-request states: [slots, *shape] float32
    summary_group: Optional[GroupStepView] = None   # paging data of the entry's block means (``CacheNeed.pool_block``): the slot
                                                    # of a token is where the mean of the block it completes goes (-1: it completes none)
    summary: Optional[torch.Tensor] = None          # [pages, kv_heads * page_size * (head_dim + value_dim)], mean keys first

    def member(self, prefix: str) -> "LayerCacheView":
        """The view of one member of a mixer made of several: the states whose names start with
        ``prefix`` + ".", under their own names."""
        cut = len(prefix) + 1
        return LayerCacheView(self.group, self.kv, self.state, self.write,
                              {k[cut:]: v for k, v in self.states.items() if k.startswith(prefix + ".")},
                              self.summary_group, self.summary)


@dataclass
class StepContext:
    num_tokens: int
    num_requests: int
    positions: torch.Tensor        # int32 [T] position of each token in its request
    tok_req: torch.Tensor          # int32 [T] row of the token's request in this step
    q_start: torch.Tensor          # int32 [R + 1] first token of each request (prefix sums of q_len)
    ctx_len: torch.Tensor          # int32 [R] tokens of the request in the cache after this step
    state_slot: torch.Tensor       # int32 [R] slot of the request's fixed-size state
    fresh: torch.Tensor            # int32 [R] 1 if this portion starts the request (state must be reset)
    groups: Dict[int, GroupStepView] = field(default_factory=dict)
    q_lens: List[int] = field(default_factory=list)       # host copies for launch decisions
    ctx_lens: List[int] = field(default_factory=list)
    host_lengths_exact: bool = False    # q_lens and ctx_lens are this step's own (not those a captured step was laid out for)
    max_q_len: int = 0
    max_ctx_len: int = 0
    attn_splits: int = 1
    tokens: Optional[torch.Tensor] = None   # int32 [T] the step's token ids (set by the model's forward pass)
    # integer lists the operator set asked for (``ops.plan_step``): name -> ``StepWork``
    work: Dict[str, Any] = field(default_factory=dict)
    # what a part of one layer leaves for parts of later layers of the same step (the results of all layers so far, ...)
    scratch: Dict[str, Any] = field(default_factory=dict)
