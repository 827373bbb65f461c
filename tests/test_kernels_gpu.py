"""Each kernel alone against a plain float32 PyTorch reference of the same operation, at
sizes other than the engine's tiny models: widths and vocabularies that are no power of
two, head sizes 48/64/128, odd group sizes, several page sizes.  Where random inputs
would hide a fault (one far key among hundreds, a window's edge, a page's edge) the
inputs are built so that it shows."""
import math

import pytest
import torch

import plain_model

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ops():
    from torchlet_b200 import ops

    return ops


def randn(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed(dtype):
    ops = _ops()
    table = randn(331, 100, dtype=dtype)
    ids = torch.tensor([0, 330, 7, 7, 100], dtype=torch.int32, device=DEV)
    acc = torch.empty(5, 100, device=DEV)
    ops.embed(table, ids, acc)
    assert torch.equal(acc, table.float()[ids.long()])


@pytest.mark.parametrize("hidden", [100, 96, 3584, 5120, 8192, 8200])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rms_norm(hidden, dtype):
    ops = _ops()
    acc, w = randn(7, hidden, scale=3.0), randn(hidden, seed=1) * 0.1 + 1
    out = torch.empty(7, hidden, device=DEV, dtype=dtype)
    ops.rms_norm(acc, w, 1e-5, out)
    want = plain_model.rms_norm(acc.cpu(), w.cpu(), 1e-5)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert (out.float().cpu() - want).abs().max() <= tol * want.abs().max()
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    picked = torch.empty(3, hidden, device=DEV, dtype=dtype)
    ops.rms_norm(acc, w, 1e-5, picked, rows)
    assert torch.equal(picked, out[rows.long()])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu(dtype):
    ops = _ops()
    gu = randn(9, 400, dtype=dtype, scale=2.0)
    out = torch.empty(9, 200, device=DEV, dtype=dtype)
    ops.swiglu(gu, out)
    g, u = gu.float()[:, :200], gu.float()[:, 200:]
    want = torch.nn.functional.silu(g) * u
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert (out.float() - want).abs().max() <= tol * want.abs().max()


@pytest.mark.parametrize("dtype, out_dtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                              (torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("M, N, K", [(1, 70, 45), (33, 130, 77), (200, 64, 256)])
def test_gemm_simt(dtype, out_dtype, M, N, K):
    ops = _ops()
    x, w, b = randn(M, K, dtype=dtype), randn(N, K, dtype=dtype, seed=1), randn(N, seed=2)
    out = torch.empty(M, N, device=DEV, dtype=out_dtype)
    ops.gemm_simt(x, w, out, b)
    want = x.double() @ w.double().t() + b.double()
    tol = 1e-5 if out_dtype == torch.float32 else 1e-2
    assert (out.double() - want).abs().max() <= tol * want.abs().max()
    if out_dtype == torch.float32:
        base = randn(M, N, seed=3)
        acc = base.clone()
        ops.gemm_simt(x, w, acc, None, accumulate=True)
        assert (acc.double() - (base.double() + want - b.double())).abs().max() <= 1e-5 * want.abs().max()
        # a row's result does not depend on the other rows of the batch
        alone = torch.empty(1, N, device=DEV)
        ops.gemm_simt(x[M - 1:], w, alone, b)
        assert torch.equal(alone[0], out[M - 1])


@pytest.mark.parametrize("M, N, K, epilogue, bias", [
    (1, 256, 128, 3, False), (8, 384, 264, 0, True), (64, 520, 1024, 1, False), (5, 448, 96, 2, False),
    (100, 1000, 520, 3, True), (300, 512, 256, 0, True), (1000, 384, 512, 1, True), (700, 448, 96, 2, False),
    (513, 1000, 72, 3, False), (257, 331, 200, 0, True), (450, 520, 264, 1, True), (200, 19200, 72, 2, False),
    # few wide tiles and a long K: the CTA-pair kernel splits K
    (200, 520, 8192, 1, True), (256, 384, 4096, 0, True), (448, 640, 2048, 2, False), (512, 300, 1544, 3, False),
])
@pytest.mark.parametrize("cta_pairs", [None, False, True])
def test_gemm_tc(M, N, K, epilogue, bias, cta_pairs):
    ops = _ops()
    if cta_pairs is not None and M <= 128:
        pytest.skip("few tokens run in the swapped orientation, which has one kernel")
    x, w = randn(M, K, dtype=torch.bfloat16, scale=0.5), randn(N, K, dtype=torch.bfloat16, scale=0.5, seed=1)
    b = randn(N, seed=2) if bias else None
    want = x.double() @ w.double().t() + (b.double() if bias else 0)
    if epilogue == ops.EPI_STORE_BF16:
        out = torch.zeros(M, N, device=DEV, dtype=torch.bfloat16)
        ops.gemm_tc(x, w, out, b, epilogue, cta_pairs=cta_pairs)
        tol = 8e-3
    elif epilogue == ops.EPI_ACCUM_F32:
        base = randn(M, N, seed=3)
        out = base.clone()
        ops.gemm_tc(x, w, out, b, epilogue, cta_pairs=cta_pairs)
        want, tol = want + base.double(), 2e-5
    elif epilogue == ops.EPI_STORE_F32:
        out = torch.zeros(M, N, device=DEV)
        ops.gemm_tc(x, w, out, b, epilogue, cta_pairs=cta_pairs)
        tol = 2e-5
    else:
        from torchlet_b200.parts.swiglu_bf16 import interleave

        inter = N // 2
        out = torch.zeros(M, inter, device=DEV, dtype=torch.bfloat16)
        ops.gemm_tc(x, interleave(w[:inter], w[inter:]), out, None, epilogue, cta_pairs=cta_pairs)
        want = torch.nn.functional.silu(want[:, :inter]) * want[:, inter:]
        tol = 8e-3
    torch.cuda.synchronize()
    assert ops.gemm_tc_error() == 0
    assert (out.double() - want).abs().max() <= tol * want.abs().max()


def test_gemm_tc_refuses_what_it_cannot_do():
    ops = _ops()
    x, w = randn(4, 100, dtype=torch.bfloat16), randn(8, 100, dtype=torch.bfloat16)
    assert not ops.gemm_tc_supported(x, w)  # K = 100 is no multiple of 8
    with pytest.raises(ops.KernelError):
        ops.gemm_tc(x, w, torch.empty(4, 8, device=DEV, dtype=torch.bfloat16))


# ----------------------------------------------------------------- attention
def paged_inputs(lens_before, q_lens, nh, nkv, d, page, dtype, seed=0, num_pages=None, shuffle=True, spike=None):
    """Random q/k/v for requests with ``lens_before`` cached tokens and ``q_lens`` new ones;
    returns the kernel's inputs and per-request dense (q, k, v) for the plain reference.
    ``spike`` = (request, new token, key position): that key is set along the token's queries
    (the first head of every group), so that one far score stands out."""
    g = torch.Generator().manual_seed(seed)
    n = len(q_lens)
    totals = [b + q for b, q in zip(lens_before, q_lens)]
    width = max(-(-t // page) for t in totals)
    need = sum(-(-t // page) for t in totals)
    num_pages = num_pages or need + 3
    order = torch.randperm(num_pages - 1, generator=g) + 1 if shuffle else torch.arange(1, num_pages)
    pages = torch.randn(num_pages, 2, nkv, page, d, generator=g).to(dtype)  # garbage everywhere first
    table = torch.zeros(n, width, dtype=torch.int32)
    dense, cursor = [], 0
    T = sum(q_lens)
    qkv = torch.zeros(T, (nh + 2 * nkv) * d, dtype=dtype)
    positions, token_req, indptr = [], [], [0]
    t0 = 0
    for i, (before, q_len, total) in enumerate(zip(lens_before, q_lens, totals)):
        k = torch.randn(total, nkv, d, generator=g).to(dtype)
        v = torch.randn(total, nkv, d, generator=g).to(dtype)
        q = torch.randn(q_len, nh, d, generator=g).to(dtype)
        if spike is not None and spike[0] == i:
            k[spike[2]] = 4 * q[spike[1], :: nh // nkv]
        count = -(-total // page)
        mine = order[cursor:cursor + count]
        cursor += count
        table[i, :count] = mine.to(torch.int32)
        for pos in range(total):
            pages[mine[pos // page], 0, :, pos % page] = k[pos]
            pages[mine[pos // page], 1, :, pos % page] = v[pos]
        qkv[t0:t0 + q_len, : nh * d] = q.reshape(q_len, nh * d)
        positions += list(range(before, total))
        token_req += [i] * q_len
        indptr.append(indptr[-1] + q_len)
        dense.append((q, k, v))
        t0 += q_len
    to = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    return dict(qkv=qkv.to(DEV), pages=pages.to(DEV), table=table.to(DEV), positions=to(positions),
                token_req=to(token_req), indptr=to(indptr), before=to(lens_before), dense=dense, T=T)


def plain_attention(dense, lens_before, nh, nkv, window, scale):
    outs = []
    for (q, k, v), before in zip(dense, lens_before):
        total = k.shape[0]
        full_q = torch.zeros(total, nh, q.shape[-1])
        full_q[before:] = q.float()
        out = plain_model.causal_gqa_attention(full_q, k.float(), v.float(), window, scale)
        outs.append(out[before:])
    return torch.cat(outs)


ATTENTION_CASES = [
    # lens_before, q_lens, nh, nkv, d, page, window
    ([0, 37, 300], [50, 1, 9], 5, 1, 48, 32, None),
    ([0, 5, 64], [33, 20, 1], 4, 2, 16, 16, 7),
    ([10, 0], [1, 130], 6, 3, 64, 8, None),
    ([700, 0, 63, 128], [1, 1, 1, 1], 14, 2, 128, 16, None),
    ([100, 90], [70, 3], 7, 1, 128, 16, 64),
]


@pytest.mark.parametrize("case", ATTENTION_CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_generic(case, dtype):
    ops = _ops()
    before, q_lens, nh, nkv, d, page, window = case
    x = paged_inputs(before, q_lens, nh, nkv, d, page, dtype)
    out = torch.zeros(x["T"], nh * d, device=DEV, dtype=dtype)
    scale = 0.37 / math.sqrt(d)
    ops.attention_generic(x["qkv"], x["qkv"].stride(0), x["pages"], x["table"], x["token_req"], x["positions"], out,
                          x["T"], nh, nkv, d, page, window, scale)
    want = plain_attention(x["dense"], before, nh, nkv, window, scale)
    tol = 2e-5 if dtype == torch.float32 else 1.5e-2
    assert (out.float().cpu() - want).abs().max() <= tol * want.abs().max()


@pytest.mark.parametrize("case", [c for c in ATTENTION_CASES if c[4] in (64, 128)] + [
    ([0], [257], 8, 8, 64, 32, None),
    ([5, 1000, 0, 17], [3, 1, 64, 1], 28, 4, 128, 16, None),
    # pages that the decode tiles' TMA boxes cannot take (larger than a key tile; not a multiple of 8): cp.async
    ([300, 40, 0], [1, 1, 5], 4, 2, 64, 128, None),
    ([33, 9], [1, 1], 6, 2, 128, 4, None),
    # a long context without key splits: three stages of key tiles
    ([1500, 2], [1, 1], 8, 2, 128, 32, 700),
])
def test_attention_mma(case):
    ops = _ops()
    before, q_lens, nh, nkv, d, page, window = case
    group = nh // nkv
    x = paged_inputs(before, q_lens, nh, nkv, d, page, torch.bfloat16, seed=3)
    scale = 0.37 / math.sqrt(d)
    want = plain_attention(x["dense"], before, nh, nkv, window, scale)
    n = len(q_lens)
    # every request through the 64-row tiles
    tile_req, tile_row = [], []
    for r, q in enumerate(q_lens):
        for start in range(0, q * group, 64):
            tile_req.append(r)
            tile_row.append(start)
    to = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    out = torch.zeros(x["T"], nh * d, device=DEV, dtype=torch.bfloat16)
    ops.attention_mma(x["qkv"], x["pages"], x["table"], x["indptr"], x["before"], to(tile_req), to(tile_row),
                      len(tile_req), out, x["T"], nh, nkv, d, page, window, scale, rows16=False)
    assert (out.float().cpu() - want).abs().max() <= 1.5e-2 * want.abs().max()
    # single-token requests through the 16-row tiles, keys split over 1, 3 and 8 CTAs
    singles = [r for r, q in enumerate(q_lens) if q == 1]
    if singles and group <= 16:
        rows = torch.tensor([sum(q_lens[:r]) for r in singles])
        # the grid holds up to ``splits`` CTAs for a request's keys; a request uses as many as its length
        # warrants; the split that finishes last merges them, or (the other mode) a second kernel does
        for splits, in_kernel in ((1, True), (3, True), (8, True), (3, False), (8, False), (64, True)):
            out2 = torch.zeros_like(out)
            saved, ops._merge_in_kernel = ops._merge_in_kernel, in_kernel
            try:
                for _ in range(2):  # twice: the arrival counters must be zero again after a launch
                    out2.zero_()
                    ops.attention_mma(x["qkv"], x["pages"], x["table"], x["indptr"], x["before"], to(singles), None,
                                      len(singles), out2, x["T"], nh, nkv, d, page, window, scale, rows16=True,
                                      splits=splits)
                    assert (out2.float().cpu()[rows] - want[rows]).abs().max() <= 1.5e-2 * want.abs().max()
            finally:
                ops._merge_in_kernel = saved
        counters = ops._arrival_counters.get(x["qkv"].device)
        assert counters is None or int(counters.abs().max()) == 0


@pytest.mark.parametrize("kernel", ["generic_f32", "generic_bf16", "mma"])
def test_attention_finds_one_far_key_and_respects_the_window_edge(kernel):
    """One key among 900 carries a large score: the output must be its value.  With a
    window, the key at the window's edge is seen and the one just outside is not."""
    ops = _ops()
    nh, nkv, d, page = 2, 1, 64, 16
    dtype = torch.float32 if kernel == "generic_f32" else torch.bfloat16
    total, far = 900, 3
    for window, hot in ((None, far), (200, total - 200), (200, total - 201)):
        k = torch.randn(total, nkv, d, generator=torch.Generator().manual_seed(1)) * 0.05
        v = torch.randn(total, nkv, d, generator=torch.Generator().manual_seed(2))
        q = torch.randn(1, nh, d, generator=torch.Generator().manual_seed(3)) * 0.05
        direction = torch.zeros(d)
        direction[5] = 1.0
        k[hot, 0] = direction * 8.0
        q[0, :] = direction * 8.0  # score 64 at the hot key, about 0 elsewhere
        num_pages = total // page + 3
        pages = torch.zeros(num_pages, 2, nkv, page, d)
        table = torch.arange(1, total // page + 2, dtype=torch.int32).flip(0).contiguous()
        for pos in range(total):
            pages[table[pos // page], 0, :, pos % page] = k[pos]
            pages[table[pos // page], 1, :, pos % page] = v[pos]
        qkv = torch.zeros(1, (nh + 2 * nkv) * d)
        qkv[0, : nh * d] = q.reshape(-1)
        to = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
        out = torch.zeros(1, nh * d, device=DEV, dtype=dtype)
        args = (qkv.to(dtype).to(DEV), pages.to(dtype).to(DEV), table.view(1, -1).to(DEV))
        if kernel == "mma":
            ops.attention_mma(args[0], args[1], args[2], to([0, 1]), to([total - 1]), None, None, 1, out, 1, nh, nkv,
                              d, page, window, 1.0, rows16=True, splits=4)
        else:
            ops.attention_generic(args[0], args[0].stride(0), args[1], args[2], to([0]), to([total - 1]), out, 1, nh,
                                  nkv, d, page, window, 1.0)
        got = out.float().cpu().view(nh, d)
        seen = window is None or hot > total - 1 - window
        if seen:
            assert (got - v[hot, 0].to(dtype).float()).abs().max() < 2e-2, (window, hot)
        else:
            assert (got - v[hot, 0]).abs().max() > 0.5, (window, hot)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d, nh, nkv, page", [(48, 5, 1, 32), (128, 4, 2, 16), (16, 2, 2, 8)])
def test_rope_and_cache_write(dtype, d, nh, nkv, page):
    ops = _ops()
    theta = 50000.0
    T = 23
    g = torch.Generator().manual_seed(0)
    qkv = torch.randn(T, (nh + 2 * nkv) * d, generator=g).to(dtype)
    positions = torch.tensor([0, 1, 2, 31, 32, 33, 400, 401] + list(range(95, 110)), dtype=torch.int32)
    token_req = torch.tensor([0] * 8 + [1] * 15, dtype=torch.int32)
    width = 402 // page + 1
    table = torch.zeros(2, width, dtype=torch.int32)
    table[0] = torch.arange(1, width + 1)
    table[1] = torch.arange(width + 1, 2 * width + 1).flip(0)
    pages = torch.zeros(2 * width + 2, 2, nkv, page, d, dtype=dtype, device=DEV)
    inv_freq = (1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).to(DEV)
    dev_qkv = qkv.to(DEV).clone()
    ops.rope_kv(dev_qkv, positions.to(DEV), token_req.to(DEV), table.to(DEV), pages, inv_freq, nh, nkv, d, page)
    x = qkv.float()
    q = plain_model.rope_split_half(x[:, : nh * d].view(T, nh, d), positions, theta)
    k = plain_model.rope_split_half(x[:, nh * d:(nh + nkv) * d].view(T, nkv, d), positions, theta)
    v = x[:, (nh + nkv) * d:].view(T, nkv, d)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    got_q = dev_qkv.float().cpu()[:, : nh * d].view(T, nh, d)
    assert (got_q - q).abs().max() <= tol * q.abs().max()
    host_pages = pages.float().cpu()
    for t in range(T):
        pos, req = int(positions[t]), int(token_req[t])
        page_id = int(table[req, pos // page])
        assert (host_pages[page_id, 0, :, pos % page] - k[t]).abs().max() <= tol * k.abs().max()
        assert torch.equal(host_pages[page_id, 1, :, pos % page], v[t])
    assert host_pages[0].abs().max() == 0  # page 0 is untouched: every token had a real page


def test_sampling_greedy_and_temperature():
    ops = _ops()
    vocab = 1531
    logits = randn(6, vocab, scale=3.0)
    logits[0, 100] = logits[0, 900] = 50.0  # a tie: the lowest index wins
    logits[1, vocab - 1] = 60.0
    out = torch.zeros(6, dtype=torch.int32, device=DEV)
    ops.sample(logits, out)
    assert out.tolist() == logits.cpu().argmax(-1).tolist() and out[0] == 100 and out[1] == vocab - 1
    temperature = torch.tensor([0.0, 0.7, 1.3, 1.3, 1.3, 2.0], device=DEV)
    seed = torch.tensor([1, 2, 3, 2, 99, 2 ** 40 + 5], dtype=torch.int64, device=DEV)
    counter = torch.tensor([0, 5, 5, 6, 5, 1], dtype=torch.int32, device=DEV)
    logits[3] = logits[2]
    logits[4] = logits[2]
    ops.sample(logits, out, temperature, seed, counter)
    host = logits.cpu()
    for r in range(6):
        if temperature[r] == 0:
            assert out[r] == host[r].argmax()
            continue
        scores = plain_model.temperature_scores(host[r], float(temperature[r]), int(seed[r]), int(counter[r]))
        best = max(scores)
        assert scores[int(out[r])] >= best - 1e-3  # the kernel's pick is the plain rule's (up to rounding)
    # same logits, same seed: the counter and the seed change the draw
    assert len({int(out[2]), int(out[3]), int(out[4])}) > 1
    again = torch.zeros_like(out)
    ops.sample(logits, again, temperature, seed, counter)
    assert torch.equal(out, again)


def test_temperature_sampling_follows_the_distribution():
    ops = _ops()
    probs = torch.tensor([0.5, 0.25, 0.125, 0.0625, 0.0625])
    rows = 4000
    logits = probs.log().repeat(rows, 1).to(DEV).contiguous()
    out = torch.zeros(rows, dtype=torch.int32, device=DEV)
    ops.sample(logits, out, torch.ones(rows, device=DEV), torch.full((rows,), 7, dtype=torch.int64, device=DEV),
               torch.arange(rows, dtype=torch.int32, device=DEV))
    freq = torch.bincount(out.long().cpu(), minlength=5).float() / rows
    assert (freq - probs).abs().max() < 0.03


def test_fused_finishing_kernels_equal_the_separate_ones():
    """finish_qkv_rope and finish_accum_norm against split finish + rope_kv / rms_norm."""
    ops = _ops()
    nh, nkv, d, page, T, H = 6, 2, 64, 16, 5, 6 * 64
    x = randn(T, H, dtype=torch.bfloat16)
    w = randn((nh + 2 * nkv) * d, H, dtype=torch.bfloat16, scale=0.1, seed=1)
    bias = randn((nh + 2 * nkv) * d, seed=2)
    positions = torch.tensor([0, 17, 300, 5, 64], dtype=torch.int32, device=DEV)
    token_req = torch.tensor([0, 0, 1, 2, 2], dtype=torch.int32, device=DEV)
    table = (torch.arange(3 * 20, dtype=torch.int32).view(3, 20) + 1).to(DEV)
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).to(DEV)
    pages_a = torch.zeros(62, 2, nkv, page, d, dtype=torch.bfloat16, device=DEV)
    pages_b = torch.zeros_like(pages_a)
    qkv_a = torch.zeros(T, (nh + 2 * nkv) * d, dtype=torch.bfloat16, device=DEV)
    ops.gemm_tc(x, w, qkv_a, bias, ops.EPI_STORE_BF16)
    ops.rope_kv(qkv_a, positions, token_req, table, pages_a, inv_freq, nh, nkv, d, page)
    partials, splits = ops.gemm_tc_deferred(x, w)
    qkv_b = torch.zeros_like(qkv_a)
    ops.finish_qkv_rope(partials, splits, bias, qkv_b, positions, token_req, table, pages_b, inv_freq, nh, nkv, d, page)
    assert torch.equal(qkv_a[:, : nh * d], qkv_b[:, : nh * d]) and torch.equal(pages_a, pages_b)

    wo = randn(H, H, dtype=torch.bfloat16, scale=0.1, seed=3)
    norm_w = randn(H, seed=4) * 0.1 + 1
    acc_a = randn(T, H, seed=5)
    acc_b = acc_a.clone()
    ops.gemm_tc(x, wo, acc_a, None, ops.EPI_ACCUM_F32)
    out_a = torch.zeros(T, H, dtype=torch.bfloat16, device=DEV)
    ops.rms_norm(acc_a, norm_w, 1e-6, out_a)
    partials, splits = ops.gemm_tc_deferred(x, wo)
    out_b = torch.zeros_like(out_a)
    ops.finish_accum_norm(partials, splits, None, acc_b, norm_w, 1e-6, out_b)
    assert (acc_a - acc_b).abs().max() <= 1e-5 * acc_a.abs().max()
    assert (out_a.float() - out_b.float()).abs().max() <= 1e-2 * out_a.float().abs().max()
    assert ops.gemm_tc_error() == 0


def test_partial_sums_of_the_pair_kernel_feed_the_fused_finishing_kernel():
    """Some hundred tokens, a narrow output and a long K: the CTA-pair kernel runs K splits and
    leaves partial sums like the few-token kernel does."""
    ops = _ops()
    T, H, K = 200, 520, 8192
    x = randn(T, K, dtype=torch.bfloat16, scale=0.5)
    w = randn(H, K, dtype=torch.bfloat16, scale=0.1, seed=1)
    _, swapped, planned = ops._gemm_plan(T, H, K)
    assert not swapped and planned > 1, "these sizes are meant to run as K splits of the pair kernel"
    partials, splits = ops.gemm_tc_deferred(x, w)
    assert splits == planned
    norm_w = randn(H, seed=4) * 0.1 + 1
    acc = randn(T, H, seed=5)
    want_acc = acc.double() + x.double() @ w.double().t()
    out = torch.zeros(T, H, dtype=torch.bfloat16, device=DEV)
    ops.finish_accum_norm(partials, splits, None, acc, norm_w, 1e-6, out)
    torch.cuda.synchronize()
    assert ops.gemm_tc_error() == 0
    assert (acc.double() - want_acc).abs().max() <= 2e-5 * want_acc.abs().max()
    want_out = want_acc * torch.rsqrt(want_acc.pow(2).mean(-1, keepdim=True) + 1e-6) * norm_w.double()
    assert (out.double() - want_out).abs().max() <= 1e-2 * want_out.abs().max()


def test_sampling_over_a_vocabulary_scanned_by_several_blocks():
    ops = _ops()
    vocab = 20011  # three chunks of 8192, the last one short
    logits = randn(5, vocab, scale=2.0, seed=9)
    logits[0, 8191] = logits[0, 8192] = 40.0  # a tie across a chunk edge: the lower index wins
    logits[1, vocab - 1] = 41.0
    out = torch.zeros(5, dtype=torch.int32, device=DEV)
    ops.sample(logits, out)
    assert out.tolist() == logits.cpu().argmax(-1).tolist() and out[0] == 8191 and out[1] == vocab - 1
    temperature = torch.tensor([0.9, 0.0, 1.5, 0.6, 1.0], device=DEV)
    seed = torch.tensor([3, 4, 5, 6, 7], dtype=torch.int64, device=DEV)
    counter = torch.tensor([0, 1, 2, 3, 4], dtype=torch.int32, device=DEV)
    ops.sample(logits, out, temperature, seed, counter)
    host = logits.cpu()
    for r in (2, 3, 4):
        scores = plain_model.temperature_scores(host[r], float(temperature[r]), int(seed[r]), int(counter[r]))
        assert scores[int(out[r])] >= max(scores) - 1e-3
    assert out[1] == vocab - 1


@pytest.mark.parametrize("case", [
    # lens_before, q_lens, nh, nkv, page, window
    ([0], [40], 7, 1, 16, None),
    ([0], [300], 28, 4, 16, None),
    ([100, 0, 700], [70, 257, 19], 14, 2, 16, None),
    ([5, 1000], [333, 40], 8, 8, 32, None),
    ([64, 0], [200, 129], 4, 2, 8, 100),
    ([0], [130], 16, 1, 128, None),
    ([0, 2500], [2, 3], 28, 4, 16, None),        # the second row tile of a CTA is empty
    ([300], [260], 4, 4, 16, 1),                # a window of the token itself: the row tiles' key ranges only touch
    ([37, 0], [500, 257], 8, 8, 32, 3),          # tiny window, one head a group: 128 tokens a row tile
    ([3000], [200], 14, 2, 16, 512),            # the row tiles start at different key tiles
    ([4000], [300], 28, 4, 64, None, (0, 299, 7)),   # a far key that decides the last token
    ([1100], [150], 12, 4, 16, 300, (0, 20, 830)),   # a key just inside the window of token 1120: 821 and later
])
@pytest.mark.parametrize("d", [128, 64])
def test_attention_tc(case, d):
    """Prompt-portion attention on tcgen05 (head_dim 128 and 64) against the plain formula."""
    ops = _ops()
    before, q_lens, nh, nkv, page, window = case[:6]
    spike = case[6] if len(case) > 6 else None
    group = nh // nkv
    assert ops.attention_tc_supported(d, group, page)
    x = paged_inputs(before, q_lens, nh, nkv, d, page, torch.bfloat16, seed=5, spike=spike)
    scale = 0.37 / math.sqrt(d)
    want = plain_attention(x["dense"], before, nh, nkv, window, scale)
    rows = ops.attention_tc_rows(group)
    assert rows == 2 * (128 // group) * group  # two row tiles of whole tokens a CTA
    tile_req, tile_row = [], []
    for r, q in enumerate(q_lens):
        for start in range(0, q * group, rows):
            tile_req.append(r)
            tile_row.append(start)
    to = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    out = torch.full((x["T"], nh * d), 7.0, device=DEV, dtype=torch.bfloat16)
    ops.attention_tc(x["qkv"], x["pages"], x["table"], x["indptr"], x["before"], to(tile_req), to(tile_row),
                     len(tile_req), out, nh, nkv, d, page, window, scale)
    torch.cuda.synchronize()
    assert ops.attention_tc_error() == 0
    assert (out.float().cpu() - want).abs().max() <= 1.5e-2 * want.abs().max()
    # the key tiles shared by two, three and five CTAs, merged by the second kernel (a workspace full of NaN first:
    # a split that sees no key of a row writes no output for it, and the merge must leave that alone)
    for splits in (2, 3, 5):
        ops._workspace(("attention_tc", x["qkv"].device), x["T"] * nh * splits * (d + 2) * 4).fill_(float("nan"))
        split_out = torch.full((x["T"], nh * d), 7.0, device=DEV, dtype=torch.bfloat16)
        ops.attention_tc(x["qkv"], x["pages"], x["table"], x["indptr"], x["before"], to(tile_req), to(tile_row),
                         len(tile_req), split_out, nh, nkv, d, page, window, scale, splits=splits,
                         token_req=x["token_req"])
        torch.cuda.synchronize()
        assert ops.attention_tc_error() == 0
        assert torch.isfinite(split_out.float()).all()
        assert (split_out.float().cpu() - want).abs().max() <= 1.5e-2 * want.abs().max(), splits
    if spike is not None:  # the spiked head's output is that key's value, in the kernel as in the formula
        token = sum(q_lens[:spike[0]]) + spike[1]
        v_spike = x["dense"][spike[0]][2][spike[2], 0].float()
        assert (want[token, :d] - v_spike).abs().max() < 0.05 * v_spike.abs().max()
        assert (out[token, :d].float().cpu() - v_spike).abs().max() < 0.05 * v_spike.abs().max()


@pytest.mark.parametrize("d", [128, 64])
@pytest.mark.parametrize("tc_splits", [1, 3])
def test_prompt_and_decode_attention_side_by_side(d, tc_splits):
    """A mixed step as the engine launches it: the prompt portions' kernel, the decode kernel right
    behind it with its wait moved to its end (it starts on the SMs the first one leaves idle), then
    the portions' deferred merge.  Every row against the plain formula, several times over, with
    the decode keys unsplit, merged inside the kernel and merged by the second kernel."""
    ops = _ops()
    nh, nkv, page = 14, 2, 16
    group = nh // nkv
    before, q_lens = [700, 0, 1500, 40, 333, 2600], [1, 90, 1, 37, 1, 1]
    x = paged_inputs(before, q_lens, nh, nkv, d, page, torch.bfloat16, seed=21)
    scale = 0.37 / math.sqrt(d)
    want = plain_attention(x["dense"], before, nh, nkv, None, scale)
    rows = ops.attention_tc_rows(group)
    tile_req, tile_row = [], []
    for r, q in enumerate(q_lens):
        if q > 1:
            for start in range(0, q * group, rows):
                tile_req.append(r)
                tile_row.append(start)
    to = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    tile_req, tile_row, decoders = to(tile_req), to(tile_row), to([0, 2, 4, 5])
    for decode_splits in (1, 4, 20):
        for _ in range(4):
            out = torch.full((x["T"], nh * d), float("nan"), device=DEV, dtype=torch.bfloat16)
            merge = ops.attention_tc(x["qkv"], x["pages"], x["table"], x["indptr"], x["before"], tile_req, tile_row,
                                     tile_req.numel(), out, nh, nkv, d, page, None, scale, splits=tc_splits,
                                     token_req=x["token_req"], defer_merge=True)
            ops.attention_mma(x["qkv"], x["pages"], x["table"], x["indptr"], x["before"], decoders, None, 4, out,
                              x["T"], nh, nkv, d, page, None, scale, rows16=True, splits=decode_splits, late_wait=True)
            assert (merge is None) == (tc_splits == 1)
            if merge is not None:
                merge()
            host = out.float().cpu()
            assert ops.attention_tc_error() == 0 and ops.attention_mma_error() == 0
            assert torch.isfinite(host).all(), (decode_splits, "a row was left unwritten")
            assert (host - want).abs().max() <= 1.5e-2 * want.abs().max(), decode_splits


# -------------------------------------------- what a kernel must leave alone, or must not be hurt by
def _poison_unowned(x, before, q_lens, page, passed=None):
    """NaN into every cache slot that no request of the step owns: page 0, pages outside every
    table (also those a window has passed: ``passed[i]`` pages of request i), and the slots of a
    request's last page past its last key."""
    pages = x["pages"]
    owned = torch.zeros(pages.shape[0], pages.shape[3], dtype=torch.bool)
    for i, (b, q) in enumerate(zip(before, q_lens)):
        for pos in range((passed[i] if passed else 0) * page, b + q):
            owned[int(x["table"][i, pos // page]), pos % page] = True
    assert not owned[0].any()
    mask = (~owned).to(pages.device)[:, None, None, :, None].expand_as(pages)
    pages[mask] = float("nan")
    return int((~owned).sum())


def test_decode_attention_beside_prompt_rows_touches_only_its_own():
    """A mixed step: two decoding requests beside two prompt portions.  The decode launch (keys
    split over CTAs, merged by a second kernel) gets ``out`` and the shared workspace full of NaN
    and a cache whose every unowned slot is NaN: it must write the two decode rows, correctly,
    and nothing else."""
    ops = _ops()
    nh, nkv, d, page = 14, 2, 128, 16
    before, q_lens = [700, 0, 333, 40], [1, 90, 1, 37]
    x = paged_inputs(before, q_lens, nh, nkv, d, page, torch.bfloat16, seed=9)
    assert _poison_unowned(x, before, q_lens, page) > 0
    scale = 0.37 / math.sqrt(d)
    want = plain_attention(x["dense"], before, nh, nkv, None, scale)
    to = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    decode_rows = [0, 91]
    for splits in (1, 4, 8):
        # a workspace of exactly the decode requests' size (2 tiles, not 129 tokens), full of NaN: a
        # kernel that wanted more would refuse the call
        exact = lambda key, nbytes: torch.full((nbytes // 4,), float("nan"), device=DEV)
        original, ops._workspace = ops._workspace, exact
        try:
            out = torch.full((x["T"], nh * d), float("nan"), device=DEV, dtype=torch.bfloat16)
            ops.attention_mma(x["qkv"], x["pages"], x["table"], x["indptr"], x["before"], to([0, 2]), None, 2, out,
                              x["T"], nh, nkv, d, page, None, scale, rows16=True, splits=splits)
        finally:
            ops._workspace = original
        host = out.float().cpu()
        others = [r for r in range(x["T"]) if r not in decode_rows]
        assert torch.isnan(host[others]).all(), f"splits {splits}: rows of other requests were written"
        assert torch.isfinite(host[decode_rows]).all(), f"splits {splits}: NaN from unowned memory reached the output"
        assert (host[decode_rows] - want[decode_rows]).abs().max() <= 1.5e-2 * want.abs().max()


@pytest.mark.parametrize("d, nh, nkv, page, window", [(128, 6, 2, 16, None), (128, 8, 2, 32, 150), (64, 14, 2, 16, None),
                                                      (64, 4, 4, 8, 70)])
def test_attention_kernels_are_not_hurt_by_nan_in_slots_they_do_not_own(d, nh, nkv, page, window):
    """Pages are never cleared when they change hands.  Prompt portions and decode tokens over a
    cache whose unowned slots (page 0, other pages, the tail of each last page) hold NaN."""
    ops = _ops()
    before, q_lens = [0, 170, 45, 301], [150, 1, 75, 1]
    group = nh // nkv
    x = paged_inputs(before, q_lens, nh, nkv, d, page, torch.bfloat16, seed=11)
    passed = [0] * len(q_lens)
    if window is not None:  # pages a window has passed are given back: their table entries name page 0
        for i, b in enumerate(before):
            passed[i] = max(0, (b + 1 - window)) // page
            x["table"][i, :passed[i]] = 0
    _poison_unowned(x, before, q_lens, page, passed)
    scale = 0.37 / math.sqrt(d)
    want = plain_attention(x["dense"], before, nh, nkv, window, scale)
    to = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    out = torch.zeros(x["T"], nh * d, device=DEV, dtype=torch.bfloat16)
    use_tc = ops.attention_tc_supported(d, group, page)
    rows = ops.attention_tc_rows(group) if use_tc else 64
    tile_req, tile_row = [], []
    for r in (0, 2):
        for start in range(0, q_lens[r] * group, rows):
            tile_req.append(r)
            tile_row.append(start)
    ops.attention_mma(x["qkv"], x["pages"], x["table"], x["indptr"], x["before"], to([1, 3]), None, 2, out, x["T"], nh,
                      nkv, d, page, window, scale, rows16=True, splits=3)
    if use_tc:
        ops.attention_tc(x["qkv"], x["pages"], x["table"], x["indptr"], x["before"], to(tile_req), to(tile_row),
                         len(tile_req), out, nh, nkv, d, page, window, scale)
    else:
        ops.attention_mma(x["qkv"], x["pages"], x["table"], x["indptr"], x["before"], to(tile_req), to(tile_row),
                          len(tile_req), out, x["T"], nh, nkv, d, page, window, scale, rows16=False)
    host = out.float().cpu()
    assert torch.isfinite(host).all(), "NaN from a slot no request owns reached an output"
    assert (host - want).abs().max() <= 1.5e-2 * want.abs().max()
    ops.raise_on_wait_errors()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_store_kv_writes_keys_and_values_unrotated(dtype):
    ops = _ops()
    nh, nkv, d, page, T = 4, 2, 32, 8, 11
    g = torch.Generator().manual_seed(4)
    qkv = torch.randn(T, (nh + 2 * nkv) * d, generator=g).to(dtype).to(DEV)
    positions = torch.tensor([0, 1, 7, 8, 9, 30, 31, 32, 33, 5, 6], dtype=torch.int32, device=DEV)
    token_req = torch.tensor([0] * 9 + [1] * 2, dtype=torch.int32, device=DEV)
    table = torch.tensor([[3, 1, 4, 6, 2], [5, 0, 0, 0, 0]], dtype=torch.int32, device=DEV)
    pages = torch.zeros(8, 2, nkv, page, d, dtype=dtype, device=DEV)
    kept = qkv.clone()
    ops.store_kv(qkv, positions, token_req, table, pages, nh, nkv, d, page)
    assert torch.equal(qkv, kept)  # q is left as it is
    for t in range(T):
        pos, req = int(positions[t]), int(token_req[t])
        page_id = int(table[req, pos // page])
        assert torch.equal(pages[page_id, 0, :, pos % page].reshape(-1), kept[t, nh * d:(nh + nkv) * d])
        assert torch.equal(pages[page_id, 1, :, pos % page].reshape(-1), kept[t, (nh + nkv) * d:])
    assert pages[0].abs().max() == 0 and pages[7].abs().max() == 0


def test_a_bounded_wait_that_runs_out_is_reported_and_the_device_stays_usable():
    """The error path of the tensor-core kernels' waits, without a fault or a hang: a block waits
    on a barrier nobody arrives at, gives up after 2^16 cycles, records its code and returns.  The
    host reads the code and raises; the code is cleared, and the next product is right."""
    ops = _ops()
    ops.raise_on_wait_errors()  # nothing pending from earlier tests
    x, w = randn(8, 256, dtype=torch.bfloat16), randn(128, 256, dtype=torch.bfloat16)
    out = torch.empty(8, 128, device=DEV, dtype=torch.bfloat16)
    ops.gemm_tc(x, w, out)  # loads the library, as the engine would have
    ops.wait_selftest(code=99)
    torch.cuda.synchronize()  # returns: the kernel ended by itself
    with pytest.raises(ops.KernelError, match="code 99"):
        ops.raise_on_wait_errors()
    ops.raise_on_wait_errors()  # reading cleared the word
    assert ops.gemm_tc_error() == 0
    ops.gemm_tc(x, w, out)
    want = x.float() @ w.float().t()
    assert (out.float() - want).abs().max() <= 1e-2 * want.abs().max()
