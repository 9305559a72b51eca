"""Each CUDA kernel alone against a plain PyTorch float32/float64 reference of the
same operation, at sizes other than the tiny models': widths and vocabularies that
are no power of two, head sizes in steps of 16, any number of heads and groups."""
import math
import random

import pytest
import torch

from plain import qwen2_plain

pytestmark = pytest.mark.gpu

DEV = "cuda"


def ops():
    from llm_serving_engine_b200.kernels import ops as kernel_ops
    return kernel_ops


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    return float((got.double() - want.double()).abs().max() / want.double().abs().max().clamp_min(1e-30))


TOL = {torch.float32: 2e-6, torch.bfloat16: 2.0 ** -8}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding(dtype):
    table = torch.randn(1000, 96, device=DEV).to(dtype)
    ids = torch.tensor([0, 999, 5, 5, 731], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 96, device=DEV)
    ops().embedding(table, ids, out)
    assert torch.equal(out, table[ids.long()].float())


@pytest.mark.parametrize("rows, hidden", [(256, 80), (300, 1536), (1000, 2048), (257, 516), (513, 1028), (256, 2052)])
@pytest.mark.parametrize("delta_dtype", [torch.float32, torch.bfloat16])
def test_add_rmsnorm_of_many_rows(rows, hidden, delta_dtype):
    """Portions of prompts (256 rows and more, bfloat16 out) take the kernel that gives a warp a row;
    widths at and beyond its limit of 2,048 included."""
    torch.manual_seed(rows + hidden)
    residual = torch.randn(rows, hidden, device=DEV) * 3
    residual[5] *= 100       # rows of very different size: every row has its own scale
    delta = torch.randn(rows, hidden, device=DEV).to(delta_dtype)
    weight = 1 + 0.1 * torch.randn(hidden, device=DEV)
    want_residual = residual.double() + delta.double()
    want = qwen2_plain.rms_norm(want_residual, weight.double(), 1e-6)
    out = torch.empty(rows, hidden, device=DEV, dtype=torch.bfloat16)
    got_residual = residual.clone()
    ops().add_rmsnorm(got_residual, delta, weight, 1e-6, out)
    assert rel_err(got_residual, want_residual) < 1e-6
    assert float(((out.double() - want).abs() / (want.abs() + 1e-3)).max()) < 2.0 ** -7


@pytest.mark.parametrize("hidden", [80, 1536, 3000])
@pytest.mark.parametrize("delta_dtype, out_dtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16)])
def test_add_rmsnorm(hidden, delta_dtype, out_dtype):
    torch.manual_seed(hidden)
    residual = torch.randn(7, hidden, device=DEV) * 3
    delta = torch.randn(7, hidden, device=DEV).to(delta_dtype)
    weight = 1 + 0.1 * torch.randn(hidden, device=DEV)
    eps = 1e-5
    want_residual = residual.double() + delta.double()
    want = qwen2_plain.rms_norm(want_residual, weight.double(), eps)
    got_residual = residual.clone()
    out = torch.empty(7, hidden, device=DEV, dtype=out_dtype)
    ops().add_rmsnorm(got_residual, delta, weight, eps, out)
    assert rel_err(got_residual, want_residual) < 1e-6        # the residual sum is float32
    assert rel_err(out, want) < TOL[out_dtype] * 2
    # no pending branch output: the residual stays as it is
    plain_out = torch.empty(7, hidden, device=DEV, dtype=out_dtype)
    keep = residual.clone()
    ops().add_rmsnorm(keep, None, weight, eps, plain_out)
    assert torch.equal(keep, residual)
    assert rel_err(plain_out, qwen2_plain.rms_norm(residual.double(), weight.double(), eps)) < TOL[out_dtype] * 2
    # selected rows only (final norm): rows are gathered, the residual is not written
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    picked = torch.empty(3, hidden, device=DEV, dtype=out_dtype)
    keep = residual.clone()
    ops().add_rmsnorm(keep, delta, weight, eps, picked, rows=rows, write_residual=False)
    assert torch.equal(keep, residual)
    assert rel_err(picked, want[rows.long()]) < TOL[out_dtype] * 2


@pytest.mark.parametrize("m, n, k", [(1, 33, 7), (5, 1000, 96), (17, 130, 1539), (70, 257, 300), (200, 64, 64)])
def test_gemm_f32_is_true_float32_and_row_invariant(m, n, k):
    torch.manual_seed(m * n)
    a = torch.randn(m, k, device=DEV)
    w = torch.randn(n, k, device=DEV)
    bias = torch.randn(n, device=DEV)
    out = torch.empty(m, n, device=DEV)
    ops().gemm_f32_nt(a, w, bias, out)
    want = a.double() @ w.double().t() + bias.double()
    # float32 accumulation over k terms: error of a few units in the last place of the sum of magnitudes
    bound = (a.abs().double() @ w.abs().double().t()) * (k * 2.0 ** -24) + 1e-6
    assert bool(((out.double() - want).abs() <= bound).all())
    # a reduced-precision product (TF32/bfloat16) would be off by about 2^-11 of the magnitudes
    assert float((out.double() - want).abs().max()) < 2.0 ** -15 * float((a.abs().double() @ w.abs().double().t()).max())
    # one row alone gives the same bits as that row inside the batch
    row = m // 2
    alone = torch.empty(1, n, device=DEV)
    ops().gemm_f32_nt(a[row:row + 1].contiguous(), w, bias, alone)
    assert torch.equal(alone[0], out[row])
    no_bias = torch.empty(m, n, device=DEV)
    ops().gemm_f32_nt(a, w, None, no_bias)
    assert rel_err(no_bias, a.double() @ w.double().t()) < 1e-5


@pytest.mark.parametrize("m, n, k", [(1, 64, 64), (8, 1536, 8960), (3, 100, 1536), (16, 257, 520), (5, 96, 4100)])
def test_gemm_f32_as_a_stack_of_range_sums(m, n, k):
    """Few rows as a stack of partial sums (a block per k range): added up in index order from zero, the stack gives
    the bits of the product that adds its ranges up itself, with few rows and as rows of a large batch."""
    torch.manual_seed(n + k)
    a = torch.randn(m, k, device=DEV)
    w = torch.randn(n, k, device=DEV)
    assert ops().gemm_f32_stack_ok(a, w)
    stack = ops().gemm_f32_stack(a, w)
    assert stack.dim() == 3 and stack.shape[1:] == (m, n) and 1 <= stack.shape[0] <= 8
    total = torch.zeros(m, n, device=DEV)
    for part in stack:
        total += part
    whole = torch.empty(m, n, device=DEV)
    ops().gemm_f32_nt(a, w, None, whole)
    assert torch.equal(total, whole)
    many = torch.randn(70, k, device=DEV)
    many[11:11 + m] = a
    large = torch.empty(70, n, device=DEV)
    ops().gemm_f32_nt(many, w, None, large)       # the many-rows kernel
    assert torch.equal(large[11:11 + m], whole)
    want = a.double() @ w.double().t()
    assert float((whole.double() - want).abs().max()) < 2.0 ** -15 * float((a.abs().double() @ w.abs().double().t()).max())
    assert not ops().gemm_f32_stack_ok(torch.randn(17, k, device=DEV), w)
    assert not ops().gemm_f32_stack_ok(torch.randn(2, 6, device=DEV), torch.randn(4, 6, device=DEV))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("head_dim, n_q, n_kv, page, pairing", [(16, 4, 2, 16, "interleaved"), (48, 10, 2, 8, "half"),
                                                             (128, 12, 2, 16, "interleaved"), (256, 3, 1, 4, "half")])
def test_rope_bias_and_cache_write(dtype, head_dim, n_q, n_kv, page, pairing):
    torch.manual_seed(head_dim)
    tokens, pages = 9, 40
    theta = 1e6
    width = (n_q + 2 * n_kv) * head_dim
    qkv = torch.randn(tokens, width, device=DEV).to(dtype)
    bias = torch.randn(width, device=DEV) * 0.1
    positions = torch.tensor([0, 1, 2, 15, 16, 17, 4095, 30000, 131071], dtype=torch.int32, device=DEV)
    slots = torch.tensor([5, 17, 0, page * pages - 1, 33, 64, 7, -1, 100], dtype=torch.int32, device=DEV)
    inv_freq = qwen2_plain.rope_inverse_frequencies(head_dim, theta).to(DEV)
    q_out = torch.zeros(tokens, n_q, head_dim, device=DEV, dtype=dtype)
    k_cache = torch.zeros(pages, n_kv, page, head_dim, device=DEV, dtype=dtype)
    v_cache = torch.zeros_like(k_cache)
    ops().rope_kv_write(qkv, bias, positions, slots, inv_freq, q_out, k_cache, v_cache, n_q, n_kv, head_dim,
                        0 if pairing == "interleaved" else 1)
    x = (qkv.float() + bias).cpu()
    q, k, v = x.split([n_q * head_dim, n_kv * head_dim, n_kv * head_dim], dim=1)
    want_q = qwen2_plain.rope(q.view(tokens, n_q, head_dim), positions.cpu(), theta, pairing)
    want_k = qwen2_plain.rope(k.view(tokens, n_kv, head_dim), positions.cpu(), theta, pairing)
    want_v = v.view(tokens, n_kv, head_dim)
    tol = 3e-5 if dtype == torch.float32 else 2.0 ** -7   # float32: sin/cos of angles up to 1e5 rad
    assert float((q_out.float().cpu() - want_q).abs().max()) < tol * float(want_q.abs().max())
    written = torch.zeros_like(k_cache, dtype=torch.bool)
    for t in range(tokens):
        slot = int(slots[t])
        if slot < 0:
            continue
        p, off = divmod(slot, page)
        assert float((k_cache[p, :, off].float().cpu() - want_k[t]).abs().max()) < tol * float(want_k.abs().max())
        assert float((v_cache[p, :, off].float().cpu() - want_v[t]).abs().max()) < tol * float(want_v.abs().max())
        written[p, :, off] = True
    assert float(k_cache[~written].abs().sum()) == 0 and float(v_cache[~written].abs().sum()) == 0  # nothing else touched
    # no bias
    q2 = torch.zeros_like(q_out)
    ops().rope_kv_write(qkv, None, positions, slots, inv_freq, q2, k_cache, v_cache, n_q, n_kv, head_dim,
                        0 if pairing == "interleaved" else 1)
    want_q2 = qwen2_plain.rope(qkv.float().cpu()[:, :n_q * head_dim].reshape(tokens, n_q, head_dim), positions.cpu(), theta, pairing)
    assert float((q2.float().cpu() - want_q2).abs().max()) < tol * float(want_q2.abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens, head_dim, n_q, n_kv, page, pairing", [
    (256, 16, 4, 2, 16, "interleaved"), (331, 48, 10, 2, 8, "half"), (300, 128, 12, 2, 16, "interleaved"),
    (277, 256, 3, 1, 4, "half"), (400, 32, 7, 7, 16, "half"), (297, 64, 33, 3, 16, "interleaved"), (64, 128, 12, 2, 16, "half")])
def test_rope_of_many_tokens(dtype, tokens, head_dim, n_q, n_kv, page, pairing):
    """Portions of prompts take the kernel that shares sines and cosines among heads: it has to
    give what the few-token kernel gives (same angles, same products) and leave padding rows alone."""
    torch.manual_seed(tokens)
    theta = 1e4
    width = (n_q + 2 * n_kv) * head_dim
    pages = (tokens + page - 1) // page + 3
    qkv = torch.randn(tokens, width, device=DEV).to(dtype)
    bias = torch.randn(width, device=DEV) * 0.1
    positions = (torch.arange(tokens, dtype=torch.int32) * 37 % 5000).to(DEV)
    order = torch.randperm(pages * page)[:tokens].to(torch.int32)
    order[5] = -1
    order[tokens - 1] = -1
    slots = order.to(DEV)
    inv_freq = qwen2_plain.rope_inverse_frequencies(head_dim, theta).to(DEV)
    code = 0 if pairing == "interleaved" else 1
    q_out = torch.zeros(tokens, n_q, head_dim, device=DEV, dtype=dtype)
    k_cache = torch.zeros(pages, n_kv, page, head_dim, device=DEV, dtype=dtype)
    v_cache = torch.zeros_like(k_cache)
    ops().rope_kv_write(qkv, bias, positions, slots, inv_freq, q_out, k_cache, v_cache, n_q, n_kv, head_dim, code)
    # the same rows, nine at a time, through the few-token kernel
    q_few = torch.zeros_like(q_out)
    k_few, v_few = torch.zeros_like(k_cache), torch.zeros_like(v_cache)
    for start in range(0, tokens, 9):
        stop = min(tokens, start + 9)
        ops().rope_kv_write(qkv[start:stop], bias, positions[start:stop], slots[start:stop], inv_freq,
                            q_few[start:stop], k_few, v_few, n_q, n_kv, head_dim, code)
    for got, few in ((q_out, q_few), (k_cache, k_few), (v_cache, v_few)):
        assert torch.equal(got, few)   # bit for bit, padding rows included
    x = (qkv.float() + bias).cpu()
    want_q = qwen2_plain.rope(x[:, :n_q * head_dim].reshape(tokens, n_q, head_dim), positions.cpu(), theta, pairing)
    tol = 3e-5 if dtype == torch.float32 else 2.0 ** -7
    assert float((q_out.float().cpu() - want_q).abs().max()) < tol * float(want_q.abs().max())


def dense_attention(q, k, v, scale, window=0):
    """q [Hq, D] at the last position of k, v [ctx, Hkv, D]; float64."""
    n_q, n_kv = q.shape[0], k.shape[1]
    ctx = k.shape[0]
    out = torch.empty_like(q, dtype=torch.float64)
    first = max(0, ctx - window) if window > 0 else 0
    for head in range(n_q):
        g = head // (n_q // n_kv)
        scores = (k[first:, g].double() @ q[head].double()) * scale
        out[head] = torch.softmax(scores, 0) @ v[first:, g].double()
    return out


def poison_unowned(k_cache, v_cache, tables, contexts, page):
    """NaN in every page that no request owns and in the unused end of every last page: none of it may
    reach a result."""
    owned = torch.zeros(k_cache.shape[0], dtype=torch.bool)
    owned[tables[tables >= 0].long().cpu()] = True
    k_cache[~owned] = float("nan")
    v_cache[~owned] = float("nan")
    for s, ctx in enumerate(contexts):
        if ctx % page:
            last = int(tables[s, (ctx - 1) // page])
            k_cache[last, :, ctx % page:] = float("nan")
            v_cache[last, :, ctx % page:] = float("nan")


def paged_setup(rng, contexts, n_kv, head_dim, page, dtype, extra_pages=5):
    """Random keys/values of each request scattered over randomly permuted physical pages."""
    need = sum(-(-c // page) for c in contexts)
    pages = need + extra_pages
    order = list(range(pages))
    rng.shuffle(order)
    k_cache = torch.randn(pages, n_kv, page, head_dim, device=DEV).to(dtype)   # unused pages hold noise
    v_cache = torch.randn(pages, n_kv, page, head_dim, device=DEV).to(dtype)
    width = max(-(-c // page) for c in contexts)
    tables = torch.full((len(contexts), width), -1, dtype=torch.int32)
    dense = []
    for s, ctx in enumerate(contexts):
        k = torch.randn(ctx, n_kv, head_dim, device=DEV).to(dtype)
        v = torch.randn(ctx, n_kv, head_dim, device=DEV).to(dtype)
        for logical in range(-(-ctx // page)):
            physical = order.pop()
            tables[s, logical] = physical
            lo, hi = logical * page, min(ctx, (logical + 1) * page)
            k_cache[physical, :, :hi - lo] = k[lo:hi].transpose(0, 1)
            v_cache[physical, :, :hi - lo] = v[lo:hi].transpose(0, 1)
        dense.append((k, v))
    return k_cache, v_cache, tables.to(DEV), dense


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("head_dim, n_q, n_kv, page", [(16, 4, 2, 16), (32, 3, 1, 8), (64, 14, 2, 1), (128, 12, 2, 16),
                                                       (128, 28, 4, 64), (256, 5, 5, 16), (80, 18, 2, 32)])
def test_paged_attention_generic(dtype, head_dim, n_q, n_kv, page):
    rng = random.Random(head_dim * n_q)
    torch.manual_seed(head_dim + n_q)
    contexts = [1, 15, 16, 17, 31, 32, 33, 65, 200, 513]
    k_cache, v_cache, tables, dense = paged_setup(rng, contexts, n_kv, head_dim, page, dtype)
    # rows: for each request its last position, and for the long ones also earlier positions (a prompt portion)
    rows = []
    for s, ctx in enumerate(contexts):
        for pos in sorted({ctx - 1, max(0, ctx - 2), ctx // 2, 0}):
            rows.append((s, pos))
    q = torch.randn(len(rows), n_q, head_dim, device=DEV).to(dtype)
    segs = torch.tensor([s for s, _ in rows], dtype=torch.int32, device=DEV)
    positions = torch.tensor([p for _, p in rows], dtype=torch.int32, device=DEV)
    out = torch.empty_like(q)
    scale = 1.0 / math.sqrt(head_dim)
    ops().paged_attention_generic(q, k_cache, v_cache, out, tables, segs, positions, scale)
    for r, (s, pos) in enumerate(rows):
        k, v = dense[s]
        want = dense_attention(q[r], k[:pos + 1], v[:pos + 1], scale)
        err = float((out[r].double() - want).abs().max())
        assert err < (1e-5 if dtype == torch.float32 else 2.0 ** -7) * max(1.0, float(want.abs().max())), (r, s, pos, err)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("needle", [0, 15, 16, 17, 255, 256, 700, 1023, 1024, 1499])
def test_one_far_key_among_hundreds_is_found(dtype, needle):
    """Random keys would hide a key that is skipped or read from the wrong page: here one
    key is made to match the query so that it takes nearly all the weight."""
    rng = random.Random(needle)
    torch.manual_seed(needle)
    n_q, n_kv, head_dim, page, ctx = 6, 2, 64, 16, 1500
    k_cache, v_cache, tables, dense = paged_setup(rng, [ctx], n_kv, head_dim, page, dtype)
    q = torch.randn(1, n_q, head_dim, device=DEV).to(dtype)
    k, v = dense[0]
    for g in range(n_kv):   # key `needle` of group g points along that group's first query head
        k[needle, g] = (q[0, g * 3].float() * 6).to(dtype)
        physical, off = int(tables[0, needle // page]), needle % page
        k_cache[physical, g, off] = k[needle, g]
    out = torch.empty_like(q)
    segs = torch.zeros(1, dtype=torch.int32, device=DEV)
    positions = torch.tensor([ctx - 1], dtype=torch.int32, device=DEV)
    ops().paged_attention_generic(q, k_cache, v_cache, out, tables, segs, positions, 1.0 / math.sqrt(head_dim))
    want = dense_attention(q[0], k, v, 1.0 / math.sqrt(head_dim))
    assert float((out[0].double() - want).abs().max()) < (1e-5 if dtype == torch.float32 else 2.0 ** -6)
    for g in range(n_kv):   # and the answer is that key's value
        assert float((out[0, g * 3].double() - v[needle, g].double()).abs().max()) < 0.05


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [0, 300])
def test_general_attention_gives_the_same_bits_with_a_block_per_chunk_of_keys(dtype, window):
    """The general kernel sums a row's keys chunk by chunk (256 keys): one block walks all chunks of its row, or every
    chunk has a block of its own and a second kernel merges them.  Rows at the edges of chunks (255, 256, 257 keys, ...),
    a far key that carries a row's weight: both ways against dense attention, and bit for bit against each other."""
    rng = random.Random(21)
    torch.manual_seed(21)
    n_q, n_kv, head_dim, page = 6, 2, 48, 8
    contexts = [1, 31, 255, 256, 257, 511, 512, 513, 700, 1025]
    k_cache, v_cache, tables, dense = paged_setup(rng, contexts, n_kv, head_dim, page, dtype)
    q = torch.randn(len(contexts), n_q, head_dim, device=DEV).to(dtype)
    needle = 3 if window == 0 else 1025 - 290     # a far key of the longest request: first chunk, or the window's first chunk
    k, v = dense[-1]
    k[needle, 1] = (q[-1, 5].float() * 6).to(dtype)
    k_cache[int(tables[-1, needle // page]), 1, needle % page] = k[needle, 1]
    poison_unowned(k_cache, v_cache, tables, contexts, page)
    segs = torch.arange(len(contexts), dtype=torch.int32, device=DEV)
    positions = torch.tensor([c - 1 for c in contexts], dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(head_dim)
    outs = []
    for split in (False, True):
        out = torch.full_like(q, 9.0)
        ops().paged_attention_generic(q, k_cache, v_cache, out, tables, segs, positions, scale, window=window, split=split)
        outs.append(out)
    assert torch.equal(outs[0], outs[1])
    bound = 1e-5 if dtype == torch.float32 else 2.0 ** -7
    for r, ctx in enumerate(contexts):
        want = dense_attention(q[r], dense[r][0][:ctx], dense[r][1][:ctx], scale, window=window)
        assert float((outs[0][r].double() - want).abs().max()) < bound * max(1.0, float(want.abs().max())), (r, ctx)
    assert float((outs[0][-1, 5].double() - v[needle, 1].double()).abs().max()) < 0.05


@pytest.mark.parametrize("window", [1, 5, 16, 33, 100])
def test_window_edge(window):
    rng = random.Random(window)
    torch.manual_seed(window)
    n_q, n_kv, head_dim, page, ctx = 4, 2, 32, 8, 120
    k_cache, v_cache, tables, dense = paged_setup(rng, [ctx], n_kv, head_dim, page, torch.float32)
    k, v = dense[0]
    rows = [3, window - 1, window, window + 1, 64, ctx - 1]
    rows = sorted({min(max(r, 0), ctx - 1) for r in rows})
    q = torch.randn(len(rows), n_q, head_dim, device=DEV)
    # the key just outside the window is made to match the query: it must NOT be read
    for r, pos in enumerate(rows):
        outside = pos - window
        if outside >= 0 and all(outside != p - window for p in rows[:r]):
            k[outside, :] = q[r, 0] * 8
            k_cache[int(tables[0, outside // page]), :, outside % page] = k[outside]
    out = torch.empty_like(q)
    segs = torch.zeros(len(rows), dtype=torch.int32, device=DEV)
    positions = torch.tensor(rows, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(head_dim)
    ops().paged_attention_generic(q, k_cache, v_cache, out, tables, segs, positions, scale, window=window)
    for r, pos in enumerate(rows):
        want = dense_attention(q[r], k[:pos + 1], v[:pos + 1], scale, window=window)
        assert float((out[r].double() - want).abs().max()) < 1e-5, (window, pos)


def test_attention_refuses_sizes_it_cannot_run():
    from llm_serving_engine_b200.kernels.library import KernelError
    q = torch.zeros(1, 2, 24, device=DEV)
    cache = torch.zeros(2, 1, 16, 24, device=DEV)
    with pytest.raises(KernelError, match="head size"):
        ops().paged_attention_generic(q, cache, cache, torch.empty_like(q), torch.zeros(1, 1, dtype=torch.int32, device=DEV),
                                      torch.zeros(1, dtype=torch.int32, device=DEV),
                                      torch.zeros(1, dtype=torch.int32, device=DEV), 1.0)
    with pytest.raises(KernelError, match="CUDA tensors only"):
        ops().silu_mul(torch.zeros(2, 4), torch.zeros(2, 2))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_silu_mul(dtype):
    gate_up = (torch.randn(13, 2 * 177, device=DEV) * 3).to(dtype)
    out = torch.empty(13, 177, device=DEV, dtype=dtype)
    ops().silu_mul(gate_up, out)
    g, u = gate_up.double()[:, :177], gate_up.double()[:, 177:]
    assert rel_err(out, torch.nn.functional.silu(g) * u) < TOL[dtype] * 2


@pytest.mark.parametrize("vocab", [7, 1000, 151936])
def test_argmax_takes_the_first_largest(vocab):
    torch.manual_seed(vocab)
    logits = torch.randn(5, vocab, device=DEV)
    logits[1, vocab // 2] = 50.0
    logits[2, vocab - 1] = 50.0
    logits[3, 3] = 50.0
    logits[3, vocab - 2] = 50.0     # a tie: the first wins
    logits[4] = -3.0                # all equal
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    ops().argmax(logits, out)
    assert out.tolist() == [int(logits[0].argmax()), vocab // 2, vocab - 1, 3, 0]


def plain_sample(logits, temperature, top_p, u):
    """Float64 restatement of the sampler: returns (token, distance of u*mass to the nearest boundary)."""
    z = logits.double() / temperature
    e = torch.exp(z - z.max())
    keep = torch.ones_like(e, dtype=torch.bool)
    if top_p < 1.0:
        order = torch.argsort(e, descending=True, stable=True)
        before = torch.cumsum(e[order], 0) - e[order]
        kept_sorted = before < top_p * e.sum()
        threshold = e[order][kept_sorted].min()
        keep = e >= threshold
    kept = torch.where(keep, e, torch.zeros_like(e))
    cdf = torch.cumsum(kept, 0)
    target = u * cdf[-1]
    token = int(torch.searchsorted(cdf, target, right=True).clamp_max(len(e) - 1))
    gap = float((cdf - target).abs().min() / cdf[-1])
    return token, gap


@pytest.mark.parametrize("vocab", [50, 1000, 151936])
def test_sampling_is_the_inverse_cdf_of_the_softmax(vocab):
    from llm_serving_engine_b200.sampling import uniform01
    torch.manual_seed(vocab)
    rows = 24
    logits = torch.randn(rows, vocab, device=DEV) * 2
    temperature = torch.tensor([0.8, 1.0, 0.3, 1.7] * 6, device=DEV)
    top_p = torch.tensor([1.0] * 12 + [0.9, 0.5, 0.8, 0.3] * 3, device=DEV)
    seed = torch.arange(rows, dtype=torch.int64, device=DEV) * 7919 + 3
    counter = torch.arange(rows, dtype=torch.int64, device=DEV) % 5
    scratch = torch.empty(rows * vocab, device=DEV)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    ops().sample(logits, temperature, top_p, seed, counter, scratch, out)
    for r in range(rows):
        u = uniform01(int(seed[r]), int(counter[r]))
        token, gap = plain_sample(logits[r].cpu(), float(temperature[r]), float(top_p[r]), u)
        assert int(out[r]) == token or gap < 1e-5, (r, int(out[r]), token, gap)
    # greedy rows inside a sampled batch take the argmax
    temperature[3] = 0.0
    ops().sample(logits, temperature, top_p, seed, counter, scratch, out)
    assert int(out[3]) == int(logits[3].argmax())


def test_sampling_follows_the_distribution():
    from llm_serving_engine_b200.sampling import uniform01
    vocab, draws = 11, 4000
    logits = torch.tensor([0.0, 1.0, 2.0, -1.0, 0.5, 3.0, -2.0, 1.5, 0.2, 2.5, -0.5], device=DEV).repeat(draws, 1)
    temperature = torch.full((draws,), 1.3, device=DEV)
    top_p = torch.ones(draws, device=DEV)
    seed = torch.full((draws,), 12345, dtype=torch.int64, device=DEV)
    counter = torch.arange(draws, dtype=torch.int64, device=DEV)
    out = torch.empty(draws, dtype=torch.int32, device=DEV)
    ops().sample(logits, temperature, top_p, seed, counter, torch.empty(draws * vocab, device=DEV), out)
    counts = torch.bincount(out.long().cpu(), minlength=vocab).double()
    probabilities = torch.softmax(logits[0].double().cpu() / 1.3, 0)
    chi2 = float(((counts - draws * probabilities) ** 2 / (draws * probabilities)).sum())
    assert chi2 < 40.0, chi2          # 10 degrees of freedom: 40 is far in the tail
    numbers = [uniform01(12345, c) for c in range(2000)]
    assert 0.47 < sum(numbers) / len(numbers) < 0.53 and min(numbers) >= 0.0 and max(numbers) < 1.0


# ------------------------------------------------------------------ tensor-core attention (bfloat16)
MMA_SHAPES = [(64, 6, 2, 16), (128, 12, 2, 16), (128, 7, 1, 8), (64, 4, 4, 1), (128, 40, 2, 64), (64, 3, 1, 32)]


@pytest.mark.parametrize("splits, cluster", [(1, True), (3, True), (8, True), (3, False), (32, False)])
@pytest.mark.parametrize("head_dim, n_q, n_kv, page", MMA_SHAPES)
def test_decode_attention_split_keys(head_dim, n_q, n_kv, page, splits, cluster):
    rng = random.Random(head_dim + n_q + splits)
    torch.manual_seed(n_q * splits)
    contexts = [1, 15, 16, 17, 63, 64, 65, 130, 1000, 2049]
    k_cache, v_cache, tables, dense = paged_setup(rng, contexts, n_kv, head_dim, page, torch.bfloat16)
    poison_unowned(k_cache, v_cache, tables, contexts, page)
    q = torch.randn(len(contexts), n_q, head_dim, device=DEV).bfloat16()
    segs = torch.arange(len(contexts), dtype=torch.int32, device=DEV)
    positions = torch.tensor([c - 1 for c in contexts], dtype=torch.int32, device=DEV)
    out = torch.empty_like(q)
    scale = 1.0 / math.sqrt(head_dim)
    assert ops().attention_mma_supported(head_dim, n_q, n_kv, torch.bfloat16)
    ops().paged_attention_decode(q, k_cache, v_cache, out, tables, segs, positions, scale, splits, cluster)
    for r, ctx in enumerate(contexts):
        k, v = dense[r]
        want = dense_attention(q[r], k, v, scale)
        err = float((out[r].double() - want).abs().max())
        assert err < 2.0 ** -7 * max(1.0, float(want.abs().max())), (r, ctx, err)
    # a padding row (segment -1) is left alone
    segs[2] = -1
    out.fill_(7.0)
    ops().paged_attention_decode(q, k_cache, v_cache, out, tables, segs, positions, scale, splits, cluster)
    assert float((out[2].float() - 7.0).abs().max()) == 0.0 and float((out[3].float() - 7.0).abs().max()) > 0.0


@pytest.mark.parametrize("needle", [0, 15, 16, 255, 256, 1023, 1024, 1499])
@pytest.mark.parametrize("splits", [1, 5])
def test_decode_attention_finds_one_far_key(needle, splits):
    rng = random.Random(needle)
    torch.manual_seed(needle)
    n_q, n_kv, head_dim, page, ctx = 12, 2, 128, 16, 1500
    k_cache, v_cache, tables, dense = paged_setup(rng, [ctx], n_kv, head_dim, page, torch.bfloat16)
    q = torch.randn(1, n_q, head_dim, device=DEV).bfloat16()
    k, v = dense[0]
    for g in range(n_kv):
        k[needle, g] = (q[0, g * 6 + 5].float() * 4).bfloat16()        # matches the last head of the group
        k_cache[int(tables[0, needle // page]), g, needle % page] = k[needle, g]
    out = torch.empty_like(q)
    ops().paged_attention_decode(q, k_cache, v_cache, out, tables, torch.zeros(1, dtype=torch.int32, device=DEV),
                                 torch.tensor([ctx - 1], dtype=torch.int32, device=DEV), 1.0 / math.sqrt(head_dim), splits)
    want = dense_attention(q[0], k, v, 1.0 / math.sqrt(head_dim))
    assert float((out[0].double() - want).abs().max()) < 2.0 ** -6
    for g in range(n_kv):
        assert float((out[0, g * 6 + 5].double() - v[needle, g].double()).abs().max()) < 0.05


@pytest.mark.parametrize("head_dim, n_q, n_kv, page", MMA_SHAPES)
def test_prefill_attention_portions_with_earlier_context(head_dim, n_q, n_kv, page):
    rng = random.Random(head_dim * n_kv + page)
    torch.manual_seed(head_dim + page)
    # (keys already cached before the portion, rows of the portion)
    portions = [(0, 1), (0, 70), (5, 2), (63, 3), (64, 64), (100, 129), (1000, 1), (300, 11), (0, 200)]
    contexts = [before + rows for before, rows in portions]
    k_cache, v_cache, tables, dense = paged_setup(rng, contexts, n_kv, head_dim, page, torch.bfloat16)
    poison_unowned(k_cache, v_cache, tables, contexts, page)
    total = sum(rows for _, rows in portions)
    q = torch.randn(total, n_q, head_dim, device=DEV).bfloat16()
    starts, firsts, cursor = [], [], 0
    for before, rows in portions:
        starts.append(cursor)
        firsts.append(before)
        cursor += rows
    starts.append(cursor)
    out = torch.empty_like(q)
    scale = 1.0 / math.sqrt(head_dim)
    ops().paged_attention_prefill(q, k_cache, v_cache, out, tables, torch.tensor(starts, dtype=torch.int32, device=DEV),
                                  torch.tensor(firsts, dtype=torch.int32, device=DEV), scale)
    for s, (before, rows) in enumerate(portions):
        k, v = dense[s]
        for local in sorted({0, 1, rows // 2, rows - 2, rows - 1} & set(range(rows))):
            pos = before + local
            want = dense_attention(q[starts[s] + local], k[:pos + 1], v[:pos + 1], scale)
            err = float((out[starts[s] + local].double() - want).abs().max())
            assert err < 2.0 ** -7 * max(1.0, float(want.abs().max())), (s, before, rows, local, err)


def test_prefill_attention_keeps_the_causal_edge():
    """The key right after a row's own position is made to match the query: it must not be read."""
    rng = random.Random(5)
    torch.manual_seed(5)
    n_q, n_kv, head_dim, page = 6, 2, 64, 16
    before, rows = 37, 150
    k_cache, v_cache, tables, dense = paged_setup(rng, [before + rows], n_kv, head_dim, page, torch.bfloat16)
    q = torch.randn(rows, n_q, head_dim, device=DEV).bfloat16()
    k, v = dense[0]
    for local in range(rows - 1):          # key pos+1 looks like the query of row `local`
        pos = before + local
        k[pos + 1, :] = (q[local, 0].float() * 4).bfloat16()
        k_cache[int(tables[0, (pos + 1) // page]), :, (pos + 1) % page] = k[pos + 1]
    out = torch.empty_like(q)
    scale = 1.0 / math.sqrt(head_dim)
    ops().paged_attention_prefill(q, k_cache, v_cache, out, tables, torch.tensor([0, rows], dtype=torch.int32, device=DEV),
                                  torch.tensor([before], dtype=torch.int32, device=DEV), scale)
    for local in (0, 1, 26, 27, 63, 64, 100, rows - 1):
        pos = before + local
        want = dense_attention(q[local], k[:pos + 1], v[:pos + 1], scale)
        assert float((out[local].double() - want).abs().max()) < 2.0 ** -6, local


def test_attention_at_the_long_context_of_the_largest_shape():
    """Five query heads a key/value head of 128, pages of 16: a 256-row portion on top of 6,144 earlier keys
    (both prompt kernels) and single rows at context 8,191 and 8,192 (the decode kernel, one and eight splits)."""
    rng = random.Random(14)
    torch.manual_seed(14)
    n_q, n_kv, head_dim, page = 10, 2, 128, 16
    scale = 1.0 / math.sqrt(head_dim)
    before, rows = 6144, 256
    k_cache, v_cache, tables, dense = paged_setup(rng, [before + rows, 8191, 8192], n_kv, head_dim, page, torch.bfloat16)
    poison_unowned(k_cache, v_cache, tables, [before + rows, 8191, 8192], page)
    q = torch.randn(rows, n_q, head_dim, device=DEV).bfloat16()
    starts = torch.tensor([0, rows], dtype=torch.int32, device=DEV)
    firsts = torch.tensor([before], dtype=torch.int32, device=DEV)
    want = dense_causal(q, dense[0][0], dense[0][1], before, scale)
    for kernel in (ops().paged_attention_prefill, ops().paged_attention_prefill_tc):
        out = torch.full_like(q, 9.0)
        kernel(q, k_cache, v_cache, out, tables, starts, firsts, scale)
        err = float((out.double() - want).abs().max())
        assert err < 2.0 ** -7 * max(1.0, float(want.abs().max())), (kernel.__name__, err)
    assert ops().attention_tc_status() == 0
    q1 = torch.randn(2, n_q, head_dim, device=DEV).bfloat16()
    segs = torch.tensor([1, 2], dtype=torch.int32, device=DEV)
    positions = torch.tensor([8190, 8191], dtype=torch.int32, device=DEV)
    for splits in (1, 8):
        out = torch.empty_like(q1)
        ops().paged_attention_decode(q1, k_cache, v_cache, out, tables, segs, positions, scale, splits)
        for r in range(2):
            want1 = dense_attention(q1[r], dense[1 + r][0], dense[1 + r][1], scale)
            assert float((out[r].double() - want1).abs().max()) < 2.0 ** -7 * max(1.0, float(want1.abs().max())), (splits, r)


def test_prompt_attention_with_more_pages_than_its_staged_block_table_holds():
    """Pages of two keys: requests of more than 1,024 pages, beside a short one, on the mma.sync prompt kernel
    (its block table no longer fits the shared-memory copy) and on the general kernel."""
    rng = random.Random(15)
    torch.manual_seed(15)
    n_q, n_kv, head_dim, page = 6, 2, 64, 2
    scale = 1.0 / math.sqrt(head_dim)
    portions = [(2300, 21), (10, 5), (2051, 70)]
    contexts = [before + rows for before, rows in portions]
    k_cache, v_cache, tables, dense = paged_setup(rng, contexts, n_kv, head_dim, page, torch.bfloat16)
    poison_unowned(k_cache, v_cache, tables, contexts, page)
    assert tables.shape[1] > 1024
    total = sum(rows for _, rows in portions)
    q = torch.randn(total, n_q, head_dim, device=DEV).bfloat16()
    starts = [0]
    for _, rows in portions:
        starts.append(starts[-1] + rows)
    out = torch.full_like(q, 9.0)
    ops().paged_attention_prefill(q, k_cache, v_cache, out, tables, torch.tensor(starts, dtype=torch.int32, device=DEV),
                                  torch.tensor([b for b, _ in portions], dtype=torch.int32, device=DEV), scale)
    segs = torch.cat([torch.full((rows,), s, dtype=torch.int32) for s, (_, rows) in enumerate(portions)]).to(DEV)
    positions = torch.cat([torch.arange(before, before + rows, dtype=torch.int32) for before, rows in portions]).to(DEV)
    general = torch.full_like(q, 9.0)
    ops().paged_attention_generic(q, k_cache, v_cache, general, tables, segs, positions, scale)
    for s, (before, rows) in enumerate(portions):
        want = dense_causal(q[starts[s]:starts[s + 1]], dense[s][0], dense[s][1], before, scale)
        for name, got in (("mma", out), ("general", general)):
            err = float((got[starts[s]:starts[s + 1]].double() - want).abs().max())
            assert err < 2.0 ** -7 * max(1.0, float(want.abs().max())), (name, s, err)


TC_SHAPES = [(128, 12, 2, 16), (64, 6, 2, 16), (128, 7, 1, 8), (64, 4, 4, 32), (128, 40, 2, 64), (64, 3, 1, 128)]


def dense_causal(q, k, v, before, scale):
    """q [rows, Hq, D] at positions before .. before+rows-1 of k, v [ctx, Hkv, D]; float64."""
    rows, n_q = q.shape[0], q.shape[1]
    group = n_q // k.shape[1]
    kk, vv = k.double().repeat_interleave(group, dim=1), v.double().repeat_interleave(group, dim=1)
    scores = torch.einsum("rhd,chd->hrc", q.double(), kk) * scale
    position = before + torch.arange(rows, device=q.device)
    hidden = torch.arange(k.shape[0], device=q.device)[None, :] > position[:, None]
    scores = scores.masked_fill(hidden[None], float("-inf"))
    return torch.einsum("hrc,chd->rhd", torch.softmax(scores, -1), vv)


@pytest.mark.parametrize("head_dim, n_q, n_kv, page", TC_SHAPES)
def test_tcgen05_prefill_attention(head_dim, n_q, n_kv, page):
    """Every row of every portion against dense attention: portions shorter and longer than a block
    of 128 rows, with and without earlier keys, starting off the tile grid; the cache pages that no
    request owns hold NaN, which must never reach a result."""
    rng = random.Random(head_dim * n_kv + page)
    torch.manual_seed(head_dim + page)
    portions = [(0, 1), (0, 70), (5, 2), (63, 3), (64, 64), (100, 129), (1000, 1), (300, 11), (0, 200), (37, 300), (128, 128)]
    contexts = [before + rows for before, rows in portions]
    k_cache, v_cache, tables, dense = paged_setup(rng, contexts, n_kv, head_dim, page, torch.bfloat16)
    owned = torch.zeros(k_cache.shape[0], dtype=torch.bool)
    owned[tables[tables >= 0].long().cpu()] = True
    k_cache[~owned] = float("nan")
    v_cache[~owned] = float("nan")
    for s, ctx in enumerate(contexts):       # so does the unused end of every last page
        if ctx % page:
            last = int(tables[s, (ctx - 1) // page])
            k_cache[last, :, ctx % page:] = float("nan")
            v_cache[last, :, ctx % page:] = float("nan")
    total = sum(rows for _, rows in portions)
    q = torch.randn(total, n_q, head_dim, device=DEV).bfloat16()
    starts = [0]
    for _, rows in portions:
        starts.append(starts[-1] + rows)
    out = torch.full_like(q, 9.0)
    scale = 1.0 / math.sqrt(head_dim)
    assert ops().attention_tc_supported(head_dim, n_q, n_kv, page, torch.bfloat16)
    ops().paged_attention_prefill_tc(q, k_cache, v_cache, out, tables, torch.tensor(starts, dtype=torch.int32, device=DEV),
                                     torch.tensor([b for b, _ in portions], dtype=torch.int32, device=DEV), scale)
    assert ops().attention_tc_status() == 0
    for s, (before, rows) in enumerate(portions):
        want = dense_causal(q[starts[s]:starts[s + 1]], dense[s][0], dense[s][1], before, scale)
        err = (out[starts[s]:starts[s + 1]].double() - want).abs()
        assert float(err.max()) < 2.0 ** -7 * max(1.0, float(want.abs().max())), (s, before, rows, float(err.max()))


@pytest.mark.parametrize("head_dim, n_q, n_kv, page, splits", [(128, 12, 2, 16, 2), (64, 6, 2, 8, 8), (128, 7, 1, 32, 1), (64, 16, 2, 16, 20)])
def test_decode_kernel_takes_the_rows_of_prompt_portions(head_dim, n_q, n_kv, page, splits):
    """Rows of prompt portions through the decode kernel, every row on its own: several rows of a request in one
    launch, each seeing the keys up to its own position, those of the earlier rows of its portion included (which
    the same step wrote: with the portions' first positions the kernel fetches none of them ahead of its wait).
    Every row against dense attention; a key right after a row's position looks like its query and must not be read."""
    rng = random.Random(head_dim + splits)
    torch.manual_seed(n_q + splits)
    portions = [(700, 40), (0, 33), (40, 1), (0, 1), (1999, 17), (15, 2), (3000, 30)]   # (keys before, rows)
    contexts = [before + rows for before, rows in portions]
    k_cache, v_cache, tables, dense = paged_setup(rng, contexts, n_kv, head_dim, page, torch.bfloat16)
    starts = [0]
    for _, rows in portions:
        starts.append(starts[-1] + rows)
    q = torch.randn(starts[-1], n_q, head_dim, device=DEV).bfloat16()
    for s, (before, rows) in enumerate(portions):   # the key after row `local` of a portion matches that row's query
        k, _ = dense[s]
        for local in range(rows - 1):
            position = before + local + 1
            k[position, :] = (q[starts[s] + local, 0].float() * 4).bfloat16()
            k_cache[int(tables[s, position // page]), :, position % page] = k[position]
    poison_unowned(k_cache, v_cache, tables, contexts, page)
    segs = torch.cat([torch.full((rows,), s, dtype=torch.int32) for s, (_, rows) in enumerate(portions)]).to(DEV)
    positions = torch.cat([torch.arange(before, before + rows, dtype=torch.int32) for before, rows in portions]).to(DEV)
    first_t = torch.tensor([before for before, _ in portions], dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(head_dim)
    out = torch.full_like(q, 9.0)
    ops().paged_attention_decode(q, k_cache, v_cache, out, tables, segs, positions, scale, splits, segment_first_position=first_t)
    for s, (before, rows) in enumerate(portions):
        want = dense_causal(q[starts[s]:starts[s + 1]], dense[s][0], dense[s][1], before, scale)
        err = float((out[starts[s]:starts[s + 1]].double() - want).abs().max())
        assert err < 2.0 ** -7 * max(1.0, float(want.abs().max())), (s, before, rows, err)


@pytest.mark.parametrize("prompt_kernel", ["tcgen05", "mma"])
@pytest.mark.parametrize("head_dim, n_q, n_kv, page, splits", [(128, 12, 2, 16, 8), (64, 6, 2, 8, 3), (128, 7, 1, 32, 1), (64, 16, 2, 16, 20)])
def test_single_tokens_beside_portions_go_to_the_decode_kernel(prompt_kernel, head_dim, n_q, n_kv, page, splits):
    """A step with prompt portions and single tokens in any order: the decode kernel, given the step's segment starts,
    works on the requests that bring one token and leaves the others alone; the prompt kernel skips exactly those.
    Every row is written once and equals dense attention; unowned pages hold NaN."""
    rng = random.Random(head_dim + n_q + splits)
    torch.manual_seed(n_q + page)
    portions = [(700, 1), (0, 130), (40, 1), (0, 1), (5, 2), (1999, 1), (300, 200), (63, 1), (0, 64)]   # (keys before, rows)
    contexts = [before + rows for before, rows in portions]
    k_cache, v_cache, tables, dense = paged_setup(rng, contexts, n_kv, head_dim, page, torch.bfloat16)
    poison_unowned(k_cache, v_cache, tables, contexts, page)
    starts = [0]
    for _, rows in portions:
        starts.append(starts[-1] + rows)
    total = starts[-1]
    q = torch.randn(total, n_q, head_dim, device=DEV).bfloat16()
    segs = torch.cat([torch.full((rows,), s, dtype=torch.int32) for s, (_, rows) in enumerate(portions)]).to(DEV)
    positions = torch.cat([torch.arange(before, before + rows, dtype=torch.int32) for before, rows in portions]).to(DEV)
    start_t = torch.tensor(starts, dtype=torch.int32, device=DEV)
    first_t = torch.tensor([before for before, _ in portions], dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(head_dim)
    out = torch.full_like(q, 9.0)
    ops().paged_attention_decode(q, k_cache, v_cache, out, tables, segs, positions, scale, splits, segment_start=start_t)
    single_rows = [starts[s] for s, (_, rows) in enumerate(portions) if rows == 1]
    untouched = torch.ones(total, dtype=torch.bool)
    untouched[single_rows] = False
    assert bool((out[untouched.to(DEV)] == 9.0).all()) and not bool((out[~untouched.to(DEV)] == 9.0).any())
    prompt = ops().paged_attention_prefill_tc if prompt_kernel == "tcgen05" else ops().paged_attention_prefill
    marked = out.clone()
    marked[~untouched.to(DEV)] = 7.0      # the prompt kernel must not write these rows again
    prompt(q, k_cache, v_cache, marked, tables, start_t, first_t, scale, skip_single=True)
    assert bool((marked[~untouched.to(DEV)] == 7.0).all()) and not bool((marked[untouched.to(DEV)] == 9.0).any())
    out[untouched.to(DEV)] = marked[untouched.to(DEV)]
    assert ops().attention_tc_status() == 0
    for s, (before, rows) in enumerate(portions):
        want = dense_causal(q[starts[s]:starts[s + 1]], dense[s][0], dense[s][1], before, scale)
        err = float((out[starts[s]:starts[s + 1]].double() - want).abs().max())
        assert err < 2.0 ** -7 * max(1.0, float(want.abs().max())), (s, before, rows, err)


@pytest.mark.parametrize("head_dim, n_q, n_kv, page, portions", [
    (128, 12, 2, 16, [(7800, 300)]),                     # a portion of a long prompt: 36 blocks, 60 key tiles each
    (64, 4, 4, 32, [(1500, 700), (0, 130)]),             # earlier keys, a ragged last block of rows, a short request beside
    (128, 7, 1, 8, [(0, 1), (3000, 128), (900, 300)]),
])
def test_tcgen05_prefill_attention_with_the_keys_of_a_tile_shared_by_several_blocks(head_dim, n_q, n_kv, page, portions):
    """Fewer blocks than SMs: several blocks take a part of the keys of a tile of rows each and the last one to arrive
    adds the parts.  Rows whose weight lies on one far key of the first part, or on one key of the last part, must
    find it; the result equals the one with every tile in one block up to rounding, and a second launch (arrival
    counters left at zero by the first) gives the same bits."""
    rng = random.Random(head_dim + page)
    torch.manual_seed(page)
    contexts = [before + rows for before, rows in portions]
    k_cache, v_cache, tables, dense = paged_setup(rng, contexts, n_kv, head_dim, page, torch.bfloat16)
    total = sum(rows for _, rows in portions)
    q = torch.randn(total, n_q, head_dim, device=DEV).bfloat16()
    starts = [0]
    for _, rows in portions:
        starts.append(starts[-1] + rows)
    needles = []
    for s, (before, rows) in enumerate(portions):
        if before + rows < 1200:
            continue
        k, v = dense[s]
        last = rows - 1
        for local, key, head in ((last, 3, 0), (last - 1, before + rows - 40, n_q - 1)):   # far in the first part; in the last part
            k[key, head // (n_q // n_kv)] = (q[starts[s] + local, head].float() * 8).bfloat16()
            k_cache[int(tables[s, key // page]), :, key % page] = k[key]
            needles.append((s, local, key, head))
    poison_unowned(k_cache, v_cache, tables, contexts, page)
    scale = 1.0 / math.sqrt(head_dim)
    start_t = torch.tensor(starts, dtype=torch.int32, device=DEV)
    first_t = torch.tensor([b for b, _ in portions], dtype=torch.int32, device=DEV)
    outs = []
    for share in (True, True, False):
        out = torch.full_like(q, 9.0)
        ops().paged_attention_prefill_tc(q, k_cache, v_cache, out, tables, start_t, first_t, scale, share_keys=share)
        assert ops().attention_tc_status() == 0
        outs.append(out)
    assert torch.equal(outs[0], outs[1])
    assert not torch.equal(outs[0], outs[2]), "no tile's keys were shared: the case does not test what it is meant to"
    assert float((outs[0].float() - outs[2].float()).abs().max()) <= 2.0 ** -7 * max(1.0, float(outs[2].float().abs().max()))
    for s, (before, rows) in enumerate(portions):
        want = dense_causal(q[starts[s]:starts[s + 1]], dense[s][0], dense[s][1], before, scale)
        err = (outs[0][starts[s]:starts[s + 1]].double() - want).abs()
        assert float(err.max()) < 2.0 ** -7 * max(1.0, float(want.abs().max())), (s, before, rows, float(err.max()))
    assert needles
    for s, local, key, head in needles:
        value = dense[s][1][key, head // (n_q // n_kv)].double()
        assert float((outs[0][starts[s] + local, head].double() - value).abs().max()) < 0.05, (s, local, key, head)


@pytest.mark.parametrize("slope", [40.0, 8.0])
def test_tcgen05_prefill_attention_when_the_maximum_grows(slope):
    """Scores that grow by far more than 2^8 from tile to tile (keys scaled up along the sequence):
    the outputs in tensor memory have to be rescaled on the way, and a far, dominant key found.
    With the steeper slope a tile's maximum lies more than 2^64 above the one in use: the tile is
    done again with the new maximum."""
    rng = random.Random(11)
    torch.manual_seed(11)
    n_q, n_kv, head_dim, page = 4, 2, 128, 16
    before, rows = 200, 700
    k_cache, v_cache, tables, dense = paged_setup(rng, [before + rows], n_kv, head_dim, page, torch.bfloat16)
    k, v = dense[0]
    q = torch.randn(rows, n_q, head_dim, device=DEV).bfloat16()
    growth = (1.0 + torch.arange(before + rows, device=DEV).float() / slope)[:, None, None]   # up to about 23 (113) times
    k[:] = (k.float().abs() * growth * q[0, 0].float().sign()).bfloat16()     # scores of row 0, head 0 rise steadily
    needle = 77                                                                 # and one early key dominates row 500
    k[needle] = (q[500, 1].float() * 6)[None, :].bfloat16()
    for position in range(before + rows):
        k_cache[int(tables[0, position // page]), :, position % page] = k[position]
    out = torch.empty_like(q)
    scale = 1.0 / math.sqrt(head_dim)
    ops().paged_attention_prefill_tc(q, k_cache, v_cache, out, tables, torch.tensor([0, rows], dtype=torch.int32, device=DEV),
                                     torch.tensor([before], dtype=torch.int32, device=DEV), scale)
    assert ops().attention_tc_status() == 0
    want = dense_causal(q, k, v, before, scale)
    err = (out.double() - want).abs()
    assert float(err.max()) < 2.0 ** -6 * max(1.0, float(want.abs().max())), float(err.max())
    if slope == 40.0:   # (with the steeper slope later keys outweigh the early one)
        assert float((out[500, 1].double() - v[needle, 0].double()).abs().max()) < 0.05


def test_tcgen05_prefill_attention_keeps_the_causal_edge():
    """The key right after a row's own position is made to match the query: it must not be read."""
    rng = random.Random(5)
    torch.manual_seed(5)
    n_q, n_kv, head_dim, page = 6, 2, 64, 16
    before, rows = 37, 300
    k_cache, v_cache, tables, dense = paged_setup(rng, [before + rows], n_kv, head_dim, page, torch.bfloat16)
    q = torch.randn(rows, n_q, head_dim, device=DEV).bfloat16()
    k, v = dense[0]
    for local in range(rows - 1):          # key pos+1 looks like the query of row `local`
        pos = before + local
        k[pos + 1, :] = (q[local, 0].float() * 4).bfloat16()
        k_cache[int(tables[0, (pos + 1) // page]), :, (pos + 1) % page] = k[pos + 1]
    out = torch.empty_like(q)
    scale = 1.0 / math.sqrt(head_dim)
    ops().paged_attention_prefill_tc(q, k_cache, v_cache, out, tables, torch.tensor([0, rows], dtype=torch.int32, device=DEV),
                                     torch.tensor([before], dtype=torch.int32, device=DEV), scale)
    want = dense_causal(q, k, v, before, scale)
    assert float((out.double() - want).abs().max()) < 2.0 ** -6


def test_tcgen05_prefill_attention_refuses_what_it_cannot_run():
    assert not ops().attention_tc_supported(80, 4, 2, 16, torch.bfloat16)
    assert not ops().attention_tc_supported(128, 4, 2, 4, torch.bfloat16)      # pages below 8 keys
    assert not ops().attention_tc_supported(128, 4, 2, 48, torch.bfloat16)     # 48 does not divide 128
    assert not ops().attention_tc_supported(128, 5, 2, 16, torch.bfloat16)
    assert not ops().attention_tc_supported(128, 4, 2, 16, torch.float32)
    assert not ops().attention_tc_supported(128, 4, 2, 16, torch.bfloat16, window=64)
    from llm_serving_engine_b200.kernels.library import KernelError
    q = torch.zeros(4, 4, 128, device=DEV, dtype=torch.bfloat16)
    cache = torch.zeros(3, 2, 4, 128, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(KernelError):
        ops().paged_attention_prefill_tc(q, cache, cache.clone(), torch.empty_like(q), torch.zeros(1, 1, dtype=torch.int32, device=DEV),
                                         torch.tensor([0, 4], dtype=torch.int32, device=DEV),
                                         torch.tensor([0], dtype=torch.int32, device=DEV), 0.1)


# ------------------------------------------------------------------ tcgen05 product and partial-sum inputs
@pytest.mark.parametrize("m, n, k, splits", [(1, 128, 64, 1), (8, 2048, 1536, 12), (3, 1536, 8960, 24), (16, 1000, 776, 3),
                                             (32, 17920, 1536, None), (7, 151936, 1536, None), (200, 384, 520, 2),
                                             (256, 130, 72, 5), (17, 96, 8, 4)])
@pytest.mark.parametrize("block_n", [128, 64])
def test_few_rows_product_on_tensor_cores(m, n, k, splits, block_n):
    torch.manual_seed(m + n + k)
    x = torch.randn(m, k, device=DEV).bfloat16()
    w = (torch.randn(n, k, device=DEV) * 0.05).bfloat16()
    parts = ops().gemm_bf16_skinny(x, w, splits, block_n=block_n)
    assert parts.dtype == torch.float32 and parts.shape[1:] == (m, n)
    got = parts.double().sum(0)
    want = x.double() @ w.double().t()
    # float32 accumulation of exact bfloat16 products
    assert bool(((got - want).abs() <= product_bound(x, w, k)).all()), float((got - want).abs().max())
    assert ops().gemm_bf16_skinny_status() == 0


def product_bound(x, w, k):
    """float32 accumulation of exact bfloat16 products."""
    return (x.abs().double() @ w.abs().double().t()) * (k * 2.0 ** -24) + 1e-6


def test_a_wait_that_runs_out_is_reported_and_the_kernel_returns():
    """Every block leaves out its last weight tile and gives up waiting for it after a few thousand tries: the kernel
    returns, the status word says so (through the synchronous read and through the copy that is queued behind a
    step's tokens), and after a reset the next launch is clean.  Nothing faults: a barrier simply gets no arrival."""
    x = torch.randn(8, 512, device=DEV).bfloat16()
    w = (torch.randn(256, 512, device=DEV) * 0.05).bfloat16()
    assert ops().gemm_bf16_skinny_status() == 0
    ops().gemm_bf16_skinny_test_hooks(spin_limit=2000, withhold=True)
    try:
        ops().gemm_bf16_skinny(x, w, 2)
        torch.cuda.synchronize()
        assert ops().gemm_bf16_skinny_status() == 1
        ops().kernel_status_reset()
        ops().gemm_bf16_skinny(x, w, 4, block_n=64)
        words = torch.zeros(2, dtype=torch.int32).pin_memory()
        ops().kernel_status_async(words)
        torch.cuda.synchronize()
        assert words.tolist() == [1, 0]
    finally:
        ops().gemm_bf16_skinny_test_hooks()
        ops().kernel_status_reset()
    got = ops().gemm_bf16_skinny(x, w).double().sum(0)
    assert bool(((got - x.double() @ w.double().t()).abs() <= product_bound(x, w, 512)).all())
    assert ops().gemm_bf16_skinny_status() == 0


def test_few_rows_product_refuses_what_it_cannot_run():
    from llm_serving_engine_b200.kernels.library import KernelError
    x = torch.randn(4, 100, device=DEV).bfloat16()      # k not a multiple of 8
    w = torch.randn(64, 100, device=DEV).bfloat16()
    assert not ops().gemm_bf16_skinny_ok(x, w)
    with pytest.raises(KernelError):
        ops().gemm_bf16_skinny(x, w)
    assert not ops().gemm_bf16_skinny_ok(torch.randn(300, 64, device=DEV).bfloat16(), torch.randn(64, 64, device=DEV).bfloat16())


@pytest.mark.parametrize("hidden", [77, 80, 1536, 9000])
def test_add_rmsnorm_of_partial_sums(hidden):
    torch.manual_seed(hidden)
    residual = torch.randn(5, hidden, device=DEV)
    partials = torch.randn(7, 5, hidden, device=DEV)
    weight = 1 + 0.1 * torch.randn(hidden, device=DEV)
    want_residual = residual.double() + partials.double().sum(0)
    want = qwen2_plain.rms_norm(want_residual, weight.double(), 1e-6)
    for out_dtype in (torch.float32, torch.bfloat16):
        got_residual = residual.clone()
        out = torch.empty(5, hidden, device=DEV, dtype=out_dtype)
        ops().add_rmsnorm(got_residual, partials, weight, 1e-6, out)
        assert rel_err(got_residual, want_residual) < 1e-6
        assert rel_err(out, want) < TOL[out_dtype] * 2
    rows = torch.tensor([4, 1], dtype=torch.int32, device=DEV)
    picked = torch.empty(2, hidden, device=DEV)
    keep = residual.clone()
    ops().add_rmsnorm(keep, partials, weight, 1e-6, picked, rows=rows, write_residual=False)
    assert torch.equal(keep, residual) and rel_err(picked, want[rows.long()]) < 4e-6


def test_rope_and_silu_of_partial_sums():
    torch.manual_seed(3)
    n_q, n_kv, head_dim, page, tokens = 12, 2, 128, 16, 6
    width = (n_q + 2 * n_kv) * head_dim
    partials = torch.randn(5, tokens, width, device=DEV)
    bias = torch.randn(width, device=DEV) * 0.1
    positions = torch.tensor([0, 3, 100, 2047, 17, 18], dtype=torch.int32, device=DEV)
    slots = torch.tensor([0, 19, 33, 5, -1, 64], dtype=torch.int32, device=DEV)
    inv_freq = qwen2_plain.rope_inverse_frequencies(head_dim, 1e6).to(DEV)
    q_out = torch.zeros(tokens, n_q, head_dim, device=DEV, dtype=torch.bfloat16)
    k_cache = torch.zeros(8, n_kv, page, head_dim, device=DEV, dtype=torch.bfloat16)
    v_cache = torch.zeros_like(k_cache)
    ops().rope_kv_write(partials, bias, positions, slots, inv_freq, q_out, k_cache, v_cache, n_q, n_kv, head_dim, 0)
    x = (partials.sum(0) + bias).cpu()
    q, k, v = x.split([n_q * head_dim, n_kv * head_dim, n_kv * head_dim], dim=1)
    want_q = qwen2_plain.rope(q.view(tokens, n_q, head_dim), positions.cpu(), 1e6)
    want_k = qwen2_plain.rope(k.view(tokens, n_kv, head_dim), positions.cpu(), 1e6)
    assert float((q_out.float().cpu() - want_q).abs().max()) < 2.0 ** -7 * float(want_q.abs().max())
    for t in (0, 1, 2, 3, 5):
        p, off = divmod(int(slots[t]), page)
        assert float((k_cache[p, :, off].float().cpu() - want_k[t]).abs().max()) < 2.0 ** -7 * float(want_k.abs().max())
        assert float((v_cache[p, :, off].float().cpu() - v.view(tokens, n_kv, head_dim)[t]).abs().max()) < 2.0 ** -7 * float(v.abs().max())
    for inter in (177, 8960):
        gate_up = torch.randn(3, 4, 2 * inter, device=DEV)
        out = torch.empty(4, inter, device=DEV, dtype=torch.bfloat16)
        ops().silu_mul(gate_up, out)
        total = gate_up.double().sum(0)
        assert rel_err(out, torch.nn.functional.silu(total[:, :inter]) * total[:, inter:]) < TOL[torch.bfloat16] * 2
