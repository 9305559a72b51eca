"""Python faces of the CUDA kernels: they check tensors and launch on the
current CUDA stream.  Every function needs CUDA tensors; there is no CPU path."""
from __future__ import annotations

import torch

from . import library
from .library import KernelError, check

F32, BF16 = 0, 1


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported dtype {dtype}: the kernels take float32 and bfloat16")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*tensors: torch.Tensor) -> None:
    for tensor in tensors:
        if tensor is not None and not tensor.is_cuda:
            raise KernelError("the kernels run on CUDA tensors only; there is no CPU fallback")


def _ptr(tensor: torch.Tensor | None) -> int | None:
    return None if tensor is None else tensor.data_ptr()


_SM_COUNT: dict = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of the device (the current one by default): launch heuristics size
    their grids by it instead of carrying one GPU's number."""
    index = torch.cuda.current_device() if device is None or torch.device(device).index is None else torch.device(device).index
    count = _SM_COUNT.get(index)
    if count is None:
        count = _SM_COUNT[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
    return count


def embedding(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t] = float32(table[ids[t]]); ids int32 [T], out float32 [T, H]."""
    _need_cuda(table, ids, out)
    vocab, hidden = table.shape
    assert ids.dtype == torch.int32 and out.dtype == torch.float32 and table.is_contiguous()
    assert out.shape == (ids.shape[0], hidden) and out.is_contiguous()
    lib = library.load()
    check(lib.lse_embedding(table.data_ptr(), dtype_code(table.dtype), ids.data_ptr(), out.data_ptr(),
                            ids.shape[0], hidden, vocab, _stream()), "embedding")
    return out


def _partials(tensor: torch.Tensor | None, rows: int, width: int):
    """(tensor, number of partial sums, elements between them) of a [rows, width] tensor or a
    float32 stack of partial sums [P, rows, width]."""
    if tensor is None:
        return None, 1, 0
    if tensor.dim() == 3:
        assert tensor.dtype == torch.float32 and tensor.shape[1:] == (rows, width) and tensor.is_contiguous()
        return tensor, tensor.shape[0], rows * width
    assert tensor.shape == (rows, width) and tensor.is_contiguous()
    return tensor, 1, 0


def add_rmsnorm(residual: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: torch.Tensor | None = None, write_residual: bool = True) -> torch.Tensor:
    """residual (+= delta); out = rmsnorm(residual) * weight.

    residual float32 [T, H]; delta [T, H] float32/bfloat16, a float32 stack of partial sums
    [P, T, H] (added in index order), or None; weight float32 [H]; out [R, H]
    float32/bfloat16 where R = len(rows) when ``rows`` (int32 row indices into residual) is
    given, else T.  With ``rows`` the residual is left unchanged unless ``write_residual``.
    """
    _need_cuda(residual, delta, weight, out, rows)
    tokens, hidden = residual.shape
    assert residual.dtype == torch.float32 and weight.dtype == torch.float32 and weight.shape == (hidden,)
    assert residual.is_contiguous() and out.is_contiguous() and out.shape[-1] == hidden
    delta, n_partials, stride = _partials(delta, tokens, hidden)
    n_rows = out.shape[0]
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.shape[0] == n_rows
    else:
        assert n_rows == tokens
    lib = library.load()
    delta_code = dtype_code(delta.dtype) if delta is not None else dtype_code(out.dtype)
    check(lib.lse_add_rmsnorm(residual.data_ptr(), _ptr(delta), delta_code, n_partials, stride, weight.data_ptr(),
                              out.data_ptr(), dtype_code(out.dtype), _ptr(rows), n_rows, hidden,
                              float(eps), int(write_residual), tokens, _stream()), "add_rmsnorm")
    return out


def gemm_f32_nt(a: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = a[M, K] @ weight[N, K]^T (+ bias[N]) in true float32."""
    _need_cuda(a, weight, bias, out)
    m, k = a.shape
    n = weight.shape[0]
    assert a.dtype == weight.dtype == out.dtype == torch.float32
    assert weight.shape[1] == k and out.shape == (m, n)
    assert a.stride(1) == 1 and weight.stride(1) == 1 and out.stride(1) == 1
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.shape == (n,)
    lib = library.load()
    check(lib.lse_gemm_f32_nt(a.data_ptr(), weight.data_ptr(), _ptr(bias), out.data_ptr(), m, n, k,
                              a.stride(0), weight.stride(0), out.stride(0), 0, 0, _stream()), "gemm_f32_nt")
    return out


def gemm_f32_stack_ok(a: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether :func:`gemm_f32_stack` takes this product (few rows, k a multiple of 4, aligned rows)."""
    return bool(library.load().lse_gemm_f32_stack_ok(a.data_ptr(), weight.data_ptr(), a.shape[0], a.shape[1],
                                                     a.stride(0), weight.stride(0)))


def gemm_f32_stack(a: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """a @ weight^T in true float32 as a stack [P, M, N] of the sums over the k ranges that the product is
    always cut into: a block per range, so that a product of few rows has enough blocks to stream the weights.
    Added up in index order, starting from zero, the stack gives :func:`gemm_f32_nt`'s result bit for bit."""
    _need_cuda(a, weight)
    m, k = a.shape
    n = weight.shape[0]
    assert a.dtype == weight.dtype == torch.float32 and weight.shape[1] == k
    assert a.stride(1) == 1 and weight.stride(1) == 1
    lib = library.load()
    ranges = int(lib.lse_gemm_f32_ranges(k))
    out = torch.empty((ranges, m, n), dtype=torch.float32, device=a.device)
    check(lib.lse_gemm_f32_nt(a.data_ptr(), weight.data_ptr(), None, out.data_ptr(), m, n, k,
                              a.stride(0), weight.stride(0), out.stride(1), 1, out.stride(0), _stream()), "gemm_f32_stack")
    return out


def rope_kv_write(qkv: torch.Tensor, bias: torch.Tensor | None, positions: torch.Tensor,
                  slot_mapping: torch.Tensor, inv_freq: torch.Tensor, q_out: torch.Tensor,
                  k_cache: torch.Tensor, v_cache: torch.Tensor, n_q: int, n_kv: int, head_dim: int,
                  pairing: int) -> None:
    """Bias, rotary encoding of queries and keys, and the write of keys and values
    into the paged cache (k_cache/v_cache: [pages, n_kv, page_size, head_dim]).
    ``qkv`` is [T, width] in the cache's dtype or in float32, or a float32 stack of
    partial sums [P, T, width]."""
    _need_cuda(qkv, bias, positions, slot_mapping, inv_freq, q_out, k_cache, v_cache)
    width = (n_q + 2 * n_kv) * head_dim
    tokens = qkv.shape[-2]
    if qkv.dim() == 3:
        qkv, n_partials, stride = _partials(qkv, tokens, width)
        row_stride = width
    else:
        assert qkv.shape[1] == width and qkv.stride(1) == 1
        n_partials, stride, row_stride = 1, 0, qkv.stride(0)
    assert positions.dtype == torch.int32 and slot_mapping.dtype == torch.int32
    assert positions.shape[0] >= tokens and slot_mapping.shape[0] >= tokens
    assert inv_freq.dtype == torch.float32 and inv_freq.shape == (head_dim // 2,)
    assert q_out.dtype == k_cache.dtype == v_cache.dtype
    assert q_out.is_contiguous() and q_out.shape == (tokens, n_q, head_dim)
    assert k_cache.is_contiguous() and v_cache.is_contiguous()
    assert k_cache.shape[1] == n_kv and k_cache.shape[3] == head_dim and v_cache.shape == k_cache.shape
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.shape == (width,)
    lib = library.load()
    check(lib.lse_rope_kv_write(qkv.data_ptr(), dtype_code(qkv.dtype), n_partials, stride, _ptr(bias),
                                positions.data_ptr(), slot_mapping.data_ptr(), inv_freq.data_ptr(),
                                q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), dtype_code(q_out.dtype),
                                tokens, n_q, n_kv, head_dim, k_cache.shape[2], pairing, row_stride, k_cache.shape[0],
                                _stream()),
          "rope_kv_write")


GENERIC_SPLIT_MAX_ROWS = 64   # up to this many rows every chunk of keys of a row gets a block of its own


def paged_attention_generic(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                            out: torch.Tensor, block_tables: torch.Tensor,
                            segment_of_token: torch.Tensor, positions: torch.Tensor, scale: float,
                            window: int = 0, split: bool | None = None) -> torch.Tensor:
    """Attention of every token of the step over its request's cached keys.

    q, out [T, n_q, D]; k_cache, v_cache [pages, n_kv, page_size, D];
    block_tables int32 [S, max_pages]; segment_of_token, positions int32 [T].
    A row's keys are summed in chunks of fixed size; ``split`` gives every chunk a block of its own
    (default: with few rows, where one block per row would leave the GPU idle).  The result does not
    depend on it, bit for bit.
    """
    _need_cuda(q, k_cache, v_cache, out, block_tables, segment_of_token, positions)
    tokens, n_q, head_dim = q.shape
    n_kv, page_size = k_cache.shape[1], k_cache.shape[2]
    if head_dim % 16 or head_dim > 256:
        raise KernelError(f"attention: head size {head_dim} is not a multiple of 16 up to 256")
    if n_q % n_kv:
        raise KernelError(f"attention: {n_q} query heads do not divide into {n_kv} groups")
    assert q.is_contiguous() and out.is_contiguous() and out.shape == q.shape
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and v_cache.shape == k_cache.shape
    assert q.dtype == out.dtype == k_cache.dtype == v_cache.dtype
    assert block_tables.dtype == torch.int32 and block_tables.dim() == 2 and block_tables.stride(1) == 1
    assert segment_of_token.dtype == torch.int32 and positions.dtype == torch.int32
    lib = library.load()
    partials, max_chunks = None, 0
    if split if split is not None else tokens <= GENERIC_SPLIT_MAX_ROWS:
        chunk = int(lib.lse_attention_generic_chunk())
        max_chunks = max(1, -(-(block_tables.stride(0) * page_size) // chunk))
        partials = torch.empty(tokens * n_q * max_chunks * (head_dim + 2), dtype=torch.float32, device=q.device)
    check(lib.lse_paged_attention_generic(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                          out.data_ptr(), dtype_code(q.dtype), block_tables.data_ptr(),
                                          block_tables.stride(0), segment_of_token.data_ptr(),
                                          positions.data_ptr(), tokens, n_q, n_kv, head_dim, page_size,
                                          float(scale), int(window), k_cache.shape[0], block_tables.shape[0],
                                          partials.data_ptr() if partials is not None else None, max_chunks,
                                          _stream()), "paged_attention_generic")
    return out


def attention_mma_supported(head_dim: int, n_q: int, n_kv: int, dtype: torch.dtype, window: int = 0) -> bool:
    """Whether the tensor-core attention kernels take this shape (bfloat16, head size 64 or 128,
    no window); other shapes run the general kernel."""
    if dtype != torch.bfloat16 or window > 0:
        return False
    return bool(library.load().lse_attention_mma_supported(head_dim, n_q, n_kv))


_DECODE_MAX_SPLITS = int(__import__("os").environ.get("LSE_DECODE_MAX_SPLITS", "8"))


_DECODE_MAX_SPLITS_LONG = 32    # the kernel's own limit


def decode_splits(tokens: int, n_q: int, n_kv: int, max_context: int | None, long_context: bool = False) -> int:
    """How many splits of the keys a decode launch uses: enough blocks to fill the GPU and a little
    more (a block that ends early makes room for the next kernel's blocks), at least one 16-key
    tile per warp and split.  (A block takes up to 8 query heads of a group.)"""
    base = tokens * n_kv * ((n_q // n_kv + 7) // 8)
    # about 1.4 blocks per SM (measured best from 12 to 64 rows on 148 SMs: 192 blocks beat 128 and 256); at most
    # 8 splits: one cluster adds them up.  Over long contexts (more than 8,192 keys) with so few rows that 8 splits
    # leave SMs without a block, more splits pay although the last-arriving block then adds them up through global
    # memory (one request of 30,000 keys: 1.60 against 2.05 ms a step; four: 1.87 against 2.13; at 8,192 keys: no gain).
    cap = _DECODE_MAX_SPLITS
    if long_context and 10 * base * cap < 7 * sm_count():
        cap = max(cap, _DECODE_MAX_SPLITS_LONG)
    splits = max(1, min(cap, ((sm_count() * 7 + 4) // 5) // base))
    if max_context is not None:
        splits = min(splits, max(1, -(-max_context // 64)))
    return splits


_ARRIVALS: dict = {}


def _arrival_counters(device, count: int) -> torch.Tensor:
    """Zeroed int32 counters that the split-KV kernel uses and leaves zero; kept per device
    so that a captured graph finds them at the same address."""
    held = _ARRIVALS.get(device)
    if held is None or held.numel() < count:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("arrival counters must exist before a stream is captured")
        held = torch.zeros(max(count, 4096), dtype=torch.int32, device=device)
        _ARRIVALS[device] = held
    return held


def paged_attention_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                           block_tables: torch.Tensor, segment_of_token: torch.Tensor, positions: torch.Tensor,
                           scale: float, num_splits: int, cluster: bool = True,
                           segment_start: torch.Tensor | None = None,
                           segment_first_position: torch.Tensor | None = None) -> torch.Tensor:
    """Attention of single decoded tokens (one row per request) with the keys split over
    ``num_splits`` blocks; bfloat16, head size 64 or 128.  With ``segment_start`` (int32 [S + 1], a step that
    also holds prompt portions) the rows are those of the requests that bring exactly one token, wherever they
    lie among q's rows; the other rows of ``out`` are left alone.  With ``segment_first_position`` (int32 [S])
    the rows may be rows of prompt portions, several of a request: every row walks its keys on its own (for
    steps of few rows, where the prompt kernels would leave most of the GPU idle)."""
    _need_cuda(q, k_cache, v_cache, out, block_tables, segment_of_token, positions)
    tokens, n_q, head_dim = q.shape
    n_kv, page_size = k_cache.shape[1], k_cache.shape[2]
    assert q.dtype == out.dtype == k_cache.dtype == v_cache.dtype == torch.bfloat16
    assert q.is_contiguous() and out.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert block_tables.dtype == torch.int32 and block_tables.stride(1) == 1
    if segment_start is not None:
        _need_cuda(segment_start)
        assert segment_start.dtype == torch.int32 and segment_start.shape[0] == block_tables.shape[0] + 1
        tokens = block_tables.shape[0]      # one block row per request of the step
    scratch = arrivals = None
    by_cluster = cluster and 1 < num_splits <= 8      # the splits add up through distributed shared memory
    if num_splits > 1 and not by_cluster:
        scratch = torch.empty(tokens * n_q * num_splits * (head_dim + 2), dtype=torch.float32, device=q.device)
        arrivals = _arrival_counters(q.device, tokens * n_kv * ((n_q // n_kv + 7) // 8))
    lib = library.load()
    check(lib.lse_paged_attention_decode(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
                                         _ptr(scratch), _ptr(arrivals), int(by_cluster), block_tables.data_ptr(),
                                         block_tables.stride(0),
                                         segment_of_token.data_ptr(), positions.data_ptr(), tokens, n_q, n_kv,
                                         head_dim, page_size, float(scale), int(num_splits), k_cache.shape[0],
                                         block_tables.shape[0], _ptr(segment_start), _ptr(segment_first_position), _stream()),
          "paged_attention_decode")
    return out


def paged_attention_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                            block_tables: torch.Tensor, segment_start: torch.Tensor,
                            segment_first_position: torch.Tensor, scale: float, skip_single: bool = False,
                            max_portions: int = 0) -> torch.Tensor:
    """Attention of prompt portions (any mix of segment lengths): causal inside the portion,
    all earlier keys of the request before it; bfloat16, head size 64 or 128.

    segment_start int32 [S + 1]: first row of each segment; segment_first_position int32 [S].
    ``skip_single``: requests that bring exactly one token are left to :func:`paged_attention_decode`;
    ``max_portions`` (with it): at most so many requests bring more than one token (it sizes the grid).
    """
    _need_cuda(q, k_cache, v_cache, out, block_tables, segment_start, segment_first_position)
    tokens, n_q, head_dim = q.shape
    n_kv, page_size = k_cache.shape[1], k_cache.shape[2]
    segments = segment_first_position.shape[0]
    assert q.dtype == out.dtype == k_cache.dtype == v_cache.dtype == torch.bfloat16
    assert q.is_contiguous() and out.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert block_tables.dtype == torch.int32 and block_tables.stride(1) == 1 and segment_start.shape[0] == segments + 1
    lib = library.load()
    check(lib.lse_paged_attention_prefill(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
                                          block_tables.data_ptr(), block_tables.stride(0), segment_start.data_ptr(),
                                          segment_first_position.data_ptr(), segments, tokens, n_q, n_kv, head_dim,
                                          page_size, float(scale), k_cache.shape[0], int(skip_single),
                                          int(max_portions) if skip_single else 0, _stream()),
          "paged_attention_prefill")
    return out


def attention_tc_supported(head_dim: int, n_q: int, n_kv: int, page_size: int, dtype: torch.dtype,
                           window: int = 0) -> bool:
    """Whether the tcgen05 prefill kernel takes this shape (bfloat16, head size 64 or 128, pages of
    8 to 128 keys that divide 128, no window)."""
    if dtype != torch.bfloat16 or window > 0:
        return False
    return bool(library.load().lse_attention_tc_supported(head_dim, n_q, n_kv, page_size))


def paged_attention_prefill_tc(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                               block_tables: torch.Tensor, segment_start: torch.Tensor,
                               segment_first_position: torch.Tensor, scale: float, skip_single: bool = False,
                               max_portions: int = 0, share_keys: bool = True) -> torch.Tensor:
    """Attention of prompt portions on the 5th-generation tensor cores: the arguments and the
    result of :func:`paged_attention_prefill`; blocks of 128 rows of one head, keys in tiles of 128
    brought in by TMA page by page, scores and outputs accumulated in tensor memory.  In a launch with fewer
    blocks than the GPU has SMs several blocks share the keys of a tile of rows; ``share_keys=False`` keeps every
    tile in one block (for comparisons)."""
    _need_cuda(q, k_cache, v_cache, out, block_tables, segment_start, segment_first_position)
    tokens, n_q, head_dim = q.shape
    pages, n_kv, page_size = k_cache.shape[0], k_cache.shape[1], k_cache.shape[2]
    segments = segment_first_position.shape[0]
    assert q.dtype == out.dtype == k_cache.dtype == v_cache.dtype == torch.bfloat16
    assert q.is_contiguous() and out.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert v_cache.shape == k_cache.shape and k_cache.shape[3] == head_dim
    assert block_tables.dtype == torch.int32 and block_tables.stride(1) == 1 and segment_start.shape[0] == segments + 1
    lib = library.load()
    scratch, counters = _attention_tc_scratch(q.device) if share_keys else (None, None)
    check(lib.lse_paged_attention_prefill_tc(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
                                             block_tables.data_ptr(), block_tables.stride(0), segment_start.data_ptr(),
                                             segment_first_position.data_ptr(), segments, tokens, pages, n_q, n_kv,
                                             head_dim, page_size, float(scale), int(skip_single),
                                             int(max_portions) if skip_single else 0, _ptr(scratch), _ptr(counters),
                                             counters.shape[0] if counters is not None else 0, _stream()),
          "paged_attention_prefill_tc")
    return out


_ATTENTION_TC_SCRATCH: dict = {}


def _attention_tc_scratch(device) -> tuple[torch.Tensor, torch.Tensor]:
    """Where the blocks of the tcgen05 prompt attention that share the keys of one tile of rows leave their parts
    (a launch with fewer blocks than SMs), and the arrival counters, which the kernel leaves at zero.  One pair per
    device, made at the first call (never inside a graph capture: a size class runs once before it is captured)."""
    index = torch.device(device).index
    index = torch.cuda.current_device() if index is None else index
    pair = _ATTENTION_TC_SCRATCH.get(index)
    if pair is None:
        slots = sm_count(index)
        floats = int(library.load().lse_attention_tc_scratch_floats())
        where = torch.device("cuda", index)
        pair = _ATTENTION_TC_SCRATCH[index] = (torch.empty(slots * floats, dtype=torch.float32, device=where),
                                               torch.zeros(slots, dtype=torch.int32, device=where))
    return pair


def attention_tc_status() -> int:
    """0 while no bounded wait of the tcgen05 attention kernel has given up (synchronises the device)."""
    return int(library.load().lse_attention_tc_status())


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t, i] = silu(gate_i) * up_i; ``gate_up`` is [T, 2I] (the row is [gate (I) | up (I)]) or a
    float32 stack of partial sums [P, T, 2I]."""
    _need_cuda(gate_up, out)
    tokens, two_i = gate_up.shape[-2], gate_up.shape[-1]
    assert two_i % 2 == 0 and out.shape == (tokens, two_i // 2) and out.is_contiguous()
    gate_up, n_partials, stride = _partials(gate_up, tokens, two_i)
    lib = library.load()
    check(lib.lse_silu_mul(gate_up.data_ptr(), dtype_code(gate_up.dtype), n_partials, stride, out.data_ptr(),
                           dtype_code(out.dtype), tokens, two_i // 2, _stream()), "silu_mul")
    return out


GEMM_SKINNY_MAX_ROWS = 256      # rows of x the few-rows product takes
_GEMM_BLOCKS_PER_SM = 2     # two blocks of the few-rows product fit on an SM; LSE_GEMM_BLOCKS overrides the total
_GEMM_MAX_SPLITS = int(__import__("os").environ.get("LSE_GEMM_MAX_SPLITS", "16"))


def _gemm_target_blocks() -> int:
    override = __import__("os").environ.get("LSE_GEMM_BLOCKS")
    return int(override) if override else _GEMM_BLOCKS_PER_SM * sm_count()


def gemm_bf16_skinny_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether the few-rows tensor-core product takes these operands."""
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.shape[0] <= GEMM_SKINNY_MAX_ROWS
            and x.shape[1] % 8 == 0 and x.is_contiguous() and weight.is_contiguous()
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def gemm_bf16_skinny(x: torch.Tensor, weight: torch.Tensor, splits: int | None = None, stages: int = 6,
                     max_splits: int | None = None, block_n: int = 128) -> torch.Tensor:
    """Partial sums [P, M, N] (float32) of x[M, K] @ weight[N, K]^T for M <= 256, bfloat16 operands;
    the k range is cut into P splits so that enough blocks stream the weights."""
    _need_cuda(x, weight)
    m, k = x.shape
    n = weight.shape[0]
    if not gemm_bf16_skinny_ok(x, weight) or weight.shape[1] != k:
        raise KernelError("gemm_bf16_skinny: operands must be contiguous bfloat16, K a multiple of 8, at most 256 rows")
    lib = library.load()
    if splits is None:
        # about two blocks per SM (more of the weights are fetched ahead while earlier kernels run), but no
        # more splits than keep the partial sums (4 bytes per row, column and split) well below the weight bytes
        n_tiles = -(-n // block_n)
        splits = 1 if n_tiles >= sm_count() else max(1, min(-(-k // 128), _gemm_target_blocks() // n_tiles,
                                                             max(1, k // (4 * m)), max_splits or _GEMM_MAX_SPLITS))
    splits = lib.lse_gemm_bf16_skinny_splits(k, int(splits))
    out = torch.empty((splits, m, n), dtype=torch.float32, device=x.device)
    check(lib.lse_gemm_bf16_skinny(x.data_ptr(), weight.data_ptr(), out.data_ptr(), m, n, k, splits, int(stages),
                                   int(block_n), _stream()), "gemm_bf16_skinny")
    return out


def gemm_bf16_skinny_test_hooks(spin_limit: int = 0, withhold: bool = False) -> None:
    """For tests of the bounded waits: ``spin_limit`` iterations before a wait gives up (0: the default),
    ``withhold``: every block leaves out its last weight tile, so that a wait runs out."""
    torch.cuda.synchronize()
    check(library.load().lse_gemm_bf16_skinny_test_hooks(int(spin_limit), int(bool(withhold))), "gemm test hooks")


def gemm_bf16_skinny_status() -> int:
    """0 unless a bounded wait inside the kernel has given up (synchronises the device)."""
    return int(library.load().lse_gemm_bf16_skinny_status())


def kernel_status_async(host_words: torch.Tensor) -> None:
    """Queue, on the current stream, copies of the status words of the kernels with bounded waits (the
    few-rows product, the tcgen05 prompt attention) into ``host_words`` (pinned int32 [2]).  Once the
    stream has got there, a non-zero word says that a wait gave up: that block wrote nothing, and
    what the step computed is not to be used."""
    assert host_words.dtype == torch.int32 and host_words.numel() >= 2 and host_words.is_pinned()
    lib = library.load()
    stream = _stream()
    if lib.lse_gemm_bf16_skinny_status_async(host_words.data_ptr(), stream) != 0 or \
            lib.lse_attention_tc_status_async(host_words.data_ptr() + 4, stream) != 0:
        raise KernelError("the kernels' status words could not be read")


def kernel_status_reset() -> None:
    """Clear both status words (after a failure has been reported)."""
    lib = library.load()
    lib.lse_gemm_bf16_skinny_status_reset()
    lib.lse_attention_tc_status_reset()
    for _, counters in _ATTENTION_TC_SCRATCH.values():   # a block that gave up may have left its arrival uncounted
        counters.zero_()


def argmax(logits: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[r] = index of the first largest value of logits[r] (float32 [R, V])."""
    _need_cuda(logits, out)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    rows, vocab = logits.shape
    lib = library.load()
    check(lib.lse_argmax(logits.data_ptr(), logits.stride(0), rows, vocab, out.data_ptr(), _stream()), "argmax")
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_p: torch.Tensor, seed: torch.Tensor,
           counter: torch.Tensor, scratch: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """Temperature / top-p sampling of one token per row (rows with temperature <= 0 take the argmax).

    temperature, top_p float32 [R]; seed, counter int64 [R]; scratch float32 with
    at least R * V values; out int32 [R].
    """
    _need_cuda(logits, temperature, top_p, seed, counter, scratch, out)
    rows, vocab = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    assert temperature.dtype == torch.float32 and top_p.dtype == torch.float32
    assert seed.dtype == torch.int64 and counter.dtype == torch.int64
    assert scratch.dtype == torch.float32 and scratch.numel() >= rows * vocab and scratch.is_contiguous()
    lib = library.load()
    check(lib.lse_sample(logits.data_ptr(), logits.stride(0), rows, vocab, temperature.data_ptr(),
                         top_p.data_ptr(), seed.data_ptr(), counter.data_ptr(), scratch.data_ptr(),
                         out.data_ptr(), _stream()), "sample")
    return out
