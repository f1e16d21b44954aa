"""What the parts see of one step: the flat batch on the device, and its geometry on the host."""

from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass
class StepContext:
    """One step's batch. All device tensors are int32 views into one arena filled by the C++
    packer and copied in a single transfer.

    Rows are requests; row r brings ``q_len[r]`` new tokens at absolute positions
    ``q_start[r] .. q_start[r] + q_len[r] - 1``; tokens of all rows are flattened in row order.
    """

    num_tokens: int  # including padding rows' tokens
    num_rows: int  # including padding rows
    num_logit_rows: int
    stream: int  # CUDA stream handle every kernel of the step is launched on
    # device, int32
    token_ids: torch.Tensor  # [T]
    positions: torch.Tensor  # [T]
    row_of_token: torch.Tensor  # [T]
    cu_q: torch.Tensor  # [R + 1] first flat token of each row
    q_start: torch.Tensor  # [R] tokens of the row already in the cache
    kv_len: torch.Tensor  # [R] tokens in the cache after this step
    state_slot: torch.Tensor  # [R] slot of the row's fixed-size state (padding rows: the spare slot no request gets)
    logit_rows: torch.Tensor  # [W] flat token indices whose logits are wanted
    page_indptr: list[torch.Tensor]  # per cache group: [R + 1]
    page_indices: list[torch.Tensor]  # per cache group: page ids, -1 where a window gave one back
    status: torch.Tensor  # [1] int32, raised by a kernel that finds inconsistent input
    # host copies of the geometry, for launch configuration and for parts written in PyTorch
    host_q_start: list[int] = field(default_factory=list)
    host_q_len: list[int] = field(default_factory=list)
    host_state_slot: list[int] = field(default_factory=list)
    max_q_len: int = 1
    max_kv_len: int = 1
    decode_only: bool = False
    leading_single_rows: int = 0  # how many rows from the front bring exactly one token (decode rows come first in a mixed step)
    sm_count: int = 148
    scratch: dict = field(default_factory=dict)  # per-step or persistent scratch buffers of kernels
    step_cache: dict = field(default_factory=dict)  # what parts compute once per step and share (e.g. the rotation table)
    buffers: dict = field(default_factory=dict)  # activation buffers of this step, by (role, shape, dtype): see buffer()
    graph_bucket: int = 0  # > 0 while a CUDA graph for this padded batch size is captured or replayed
    graph_kv_len: int = 0  # inside a decode graph: the context length its launches are laid out for (0: a few thousand keys)
    # Set while a pass is captured as a chain of CUDA graphs (engine/graphs.py, StepGraphs): an operation whose
    # launches depend on how the step's tokens are shared among rows hands itself to ``recorder.defer``
    # instead of launching; it is then called with each later step's context, between the graphs.
    recorder: object | None = None
    layout: tuple = ()  # where each field starts in the arena (a replayed graph checks it has not moved)

    def buffer(self, role: str, shape: tuple, dtype: torch.dtype, device) -> torch.Tensor:
        """An uninitialised activation tensor that lives for one pass of the model over this step
        (the model empties ``buffers`` when a pass begins) and is shared by every layer: the first caller with this (role, shape, dtype) allocates it, later callers get the
        same tensor. Kernels of one step run in stream order, so a part may take a role's buffer
        again in the next layer once nothing of its own still reads it. A part names a role for
        each tensor it has alive at the same time ("attn.qkv", "attn.q", ...)."""
        key = (role, shape, dtype)
        t = self.buffers.get(key)
        if t is None:
            t = torch.empty(shape, dtype=dtype, device=device)
            self.buffers[key] = t
        return t
