"""Grouped-query attention over the paged cache
(reference ``src/llmserve/model.py:46-177``)."""
from __future__ import annotations

import math
import os

import torch

from ..kernels import ops
from ..weights.tensor_spec import TensorSpec
from .base import POSITION_ENCODINGS, Mixer, PagedKV, register_mixer
from .linear import linear_partials

# Which kernels a step with prompt portions takes.  Requests that bring a single token (decoding requests beside
# the portions, a prompt's last token) go to the decode kernel, which splits their keys over blocks; the portions
# go to one of the two prompt kernels.  The tcgen05 kernel's block is 128 rows of one request and one head; the
# mma.sync kernel's about ten rows of all heads of a group.  The portions go to the former when the longest has at
# least TCGEN05_MIN_ROWS (64) rows and either their blocks fit the GPU at once or they are long on average (at least 64
# rows each); many short portions stay on the mma.sync kernel.  LSE_PREFILL_ATTENTION=mma turns the tcgen05
# kernel off, LSE_MIXED_DECODE_KERNEL=0 sends single tokens through the prompt kernels as well.
TCGEN05_MIN_ROWS = int(os.environ.get("LSE_TCGEN05_MIN_ROWS", "64"))
TCGEN05_MIN_ROWS_PER_REQUEST = 64
TCGEN05_PREFILL = os.environ.get("LSE_PREFILL_ATTENTION", "tcgen05") != "mma"
MIXED_DECODE_KERNEL = os.environ.get("LSE_MIXED_DECODE_KERNEL", "1") != "0"
# A step of fewer rows than this (portions and single tokens together) goes to the decode kernel row by row: a prompt
# kernel would have a handful of blocks, each walking all keys of its request (16 rows on 8,000 earlier keys: 21 against
# 150 us on the mma.sync kernel; on 200 keys no difference).  From 64 rows on the tcgen05 kernel, whose blocks share the
# keys of a tile, is as fast or faster (portions of 32 / 64 / 96 tokens of an 8,192-token prompt: 1.58 / 2.13 / 2.68 ms a
# step row by row, 1.85 / 2.15 / 2.07 on the tcgen05 kernel).  LSE_ROWS_KERNEL_BELOW=0 turns it off.
ROWS_KERNEL_BELOW = int(os.environ.get("LSE_ROWS_KERNEL_BELOW", "64"))
ROWS_KERNEL_BLOCKS = 256


@register_mixer("gqa_attention")
class GroupedQueryAttention(Mixer):
    """params: ``num_heads``, ``num_kv_heads``, ``head_dim``, ``bias`` (on q/k/v),
    ``window`` (0 = all keys), ``position`` (a PartSpec-like dict: kind, params).

    Tensors: ``q_proj/k_proj/v_proj.weight`` (+ ``.bias``), ``o_proj.weight``; the
    three projections are stacked into one matrix when the part is built.
    Every row of the step writes its key and value first, then attends to the
    keys of its own request up to its own position, scaled by 1/sqrt(head_dim).
    """

    graph_safe = True

    def __init__(self, params, weights, ctx) -> None:
        super().__init__(params, weights, ctx)
        self.n_q = int(params["num_heads"])
        self.n_kv = int(params["num_kv_heads"])
        self.head_dim = int(params["head_dim"])
        self.window = int(params.get("window", 0))
        self.scale = 1.0 / math.sqrt(self.head_dim)
        if self.head_dim % 16 or self.head_dim > 256:
            raise ops.KernelError(
                f"attention: head size {self.head_dim} is not supported (multiples of 16 up to 256)")
        self.qkv_weight = torch.cat(
            [weights["q_proj.weight"], weights["k_proj.weight"], weights["v_proj.weight"]], dim=0).contiguous()
        self.qkv_bias = None
        if params.get("bias", True):
            self.qkv_bias = torch.cat(
                [weights["q_proj.bias"], weights["k_proj.bias"], weights["v_proj.bias"]]).float().contiguous()
        self.o_weight = weights["o_proj.weight"].contiguous()
        position = params["position"]
        self.position = POSITION_ENCODINGS.get(position["kind"])(position["params"], {}, ctx)

    @classmethod
    def expected_tensors(cls, params, hidden_size):
        n_q, n_kv, d = int(params["num_heads"]), int(params["num_kv_heads"]), int(params["head_dim"])
        out = {
            "q_proj.weight": TensorSpec((n_q * d, hidden_size)),
            "k_proj.weight": TensorSpec((n_kv * d, hidden_size)),
            "v_proj.weight": TensorSpec((n_kv * d, hidden_size)),
            "o_proj.weight": TensorSpec((hidden_size, n_q * d)),
        }
        if params.get("bias", True):
            out["q_proj.bias"] = TensorSpec((n_q * d,), "bias")
            out["k_proj.bias"] = TensorSpec((n_kv * d,), "bias")
            out["v_proj.bias"] = TensorSpec((n_kv * d,), "bias")
        return out

    @classmethod
    def cache_requirement(cls, params, hidden_size):
        return PagedKV(int(params["num_kv_heads"]), int(params["head_dim"]), int(params.get("window", 0)))

    def prompt_kernel(self, segment_counts: list[int], page_size: int | None = None) -> str:
        """"tcgen05" or "mma": the kernel a step with prompt portions takes (the rule at the top of this file)."""
        if not TCGEN05_PREFILL or max(segment_counts) < TCGEN05_MIN_ROWS:
            return "mma"
        long_on_average = sum(segment_counts) >= TCGEN05_MIN_ROWS_PER_REQUEST * len(segment_counts)
        blocks_at_once = sum(-(-count // 128) for count in segment_counts) * self.n_q <= ops.sm_count()
        if not (long_on_average or blocks_at_once):
            return "mma"
        if page_size is not None and not ops.attention_tc_supported(self.head_dim, self.n_q, self.n_kv, page_size,
                                                                    self.ctx.dtype, self.window):
            return "mma"
        return "tcgen05"

    @staticmethod
    def _portions(segment_counts: list[int]) -> tuple[list[int], bool]:
        """The portions that the prompt kernel takes, and whether the decode kernel takes the single tokens."""
        singles = MIXED_DECODE_KERNEL and any(count == 1 for count in segment_counts) and max(segment_counts) > 1
        return ([count for count in segment_counts if count > 1] if singles else list(segment_counts)), singles

    PORTION_CLASSES = (2, 16)   # beside single tokens: at most so many portions (it sizes the prompt kernel's grid)

    def _portion_class(self, portions: list[int], singles: bool) -> int:
        """An upper bound on the number of portions that a step of this kind holds beside its single tokens (0: no bound)."""
        if not singles:
            return 0
        return next((bound for bound in self.PORTION_CLASSES if bound >= len(portions)), 0)

    def launch_signature(self, segment_counts):
        if max(segment_counts) == 1 or not ops.attention_mma_supported(self.head_dim, self.n_q, self.n_kv, self.ctx.dtype, self.window):
            return ()
        if sum(segment_counts) < ROWS_KERNEL_BELOW:
            return ("rows",)
        portions, singles = self._portions(segment_counts)
        return (self.prompt_kernel(portions), singles, self._portion_class(portions, singles))

    def forward(self, x, step, cache):
        tokens = x.shape[0]
        # bias is added with the rotation, in float32; at most 8 partial sums: the rotary kernel fetches them in one go
        qkv = linear_partials(x, self.qkv_weight, max_splits=8)
        q = torch.empty((tokens, self.n_q, self.head_dim), dtype=x.dtype, device=x.device)
        self.position.encode_and_store(qkv, self.qkv_bias, step, cache, q, self.n_q, self.n_kv, self.head_dim)
        attended = torch.empty_like(q)
        if ops.attention_mma_supported(self.head_dim, self.n_q, self.n_kv, x.dtype, self.window):
            if step.decode_only:
                splits = ops.decode_splits(tokens, self.n_q, self.n_kv, step.max_context, getattr(step, "long_context", False))
                ops.paged_attention_decode(q, cache.keys, cache.values, attended, cache.block_tables,
                                           step.segment_of_token, step.positions, self.scale, splits)
            elif sum(segment.count for segment in step.segments) < ROWS_KERNEL_BELOW:
                # few rows: every row walks its keys on its own, split over blocks (256 blocks or so), as in a decode step
                blocks_a_split = tokens * self.n_kv * ((self.n_q // self.n_kv + 7) // 8)
                ops.paged_attention_decode(q, cache.keys, cache.values, attended, cache.block_tables,
                                           step.segment_of_token, step.positions, self.scale,
                                           max(1, min(8, ROWS_KERNEL_BLOCKS // blocks_a_split)),
                                           segment_first_position=step.segment_first_position)
            else:
                portions, singles = self._portions([segment.count for segment in step.segments])
                if singles:   # one block row per request of the step; requests with portions leave at once
                    requests = cache.block_tables.shape[0]
                    splits = ops.decode_splits(requests, self.n_q, self.n_kv, None)
                    ops.paged_attention_decode(q, cache.keys, cache.values, attended, cache.block_tables,
                                               step.segment_of_token, step.positions, self.scale, splits,
                                               segment_start=step.segment_start)
                prompt = (ops.paged_attention_prefill_tc if self.prompt_kernel(portions, cache.keys.shape[2]) == "tcgen05"
                          else ops.paged_attention_prefill)
                prompt(q, cache.keys, cache.values, attended, cache.block_tables, step.segment_start,
                       step.segment_first_position, self.scale, skip_single=singles,
                       max_portions=self._portion_class(portions, singles))
        else:   # float32, other head sizes, windows: the general kernel
            ops.paged_attention_generic(q, cache.keys, cache.values, attended, cache.block_tables,
                                        step.segment_of_token, step.positions, self.scale, self.window)
        return linear_partials(attended.view(tokens, self.n_q * self.head_dim), self.o_weight)
