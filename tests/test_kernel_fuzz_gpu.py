"""Seeded random sizes through the tensor-core kernels, each against a float64 restatement:
the tcgen05 product over token counts, widths and depths on every side of its plans (few and many
tokens, K splits, single CTAs and CTA pairs, every epilogue), and the two attention kernels of a
mixed step launched side by side over random head geometries, page sizes, windows, cached lengths
and key splits."""
import math
import random

import pytest
import torch

import test_kernels_gpu as kernels

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("seed", [1, 2])
def test_products_of_random_sizes(seed):
    from torchlet_b200 import ops

    rng = random.Random(seed)
    for trial in range(60):
        M = rng.choice([1, 2, 7, 8, 15, 16, 17, 31, 33, 63, 64, 65, 100, 127, 128, 129, 200, 255, 256, 257, 300, 511, 512,
                        513, 700, 1025])
        N = rng.choice([8, 24, 40, 120, 128, 136, 256, 264, 1000, 1152, 2048, 3584, 4608, 5000, 9728])
        K = rng.choice([8, 16, 64, 72, 128, 200, 512, 896, 1000, 3584, 4864, 5120])
        epilogue = rng.choice(["bf16", "f32", "accum", "swiglu"])
        if epilogue == "swiglu" and N % 32:
            N = (N // 32 + 1) * 32
        g = torch.Generator(device=DEV).manual_seed(1000 * seed + trial)
        x = (torch.randn(M, K, device=DEV, generator=g) * 0.5).bfloat16()
        w = (torch.randn(N, K, device=DEV, generator=g) * 0.1).bfloat16()
        bias = torch.randn(N, device=DEV, generator=g) * 0.1 if epilogue in ("bf16", "f32") and rng.random() < 0.5 else None
        want = x.double() @ w.double().t() + (bias.double() if bias is not None else 0.0)
        if epilogue == "bf16":
            out = torch.full((M, N), 7.0, device=DEV, dtype=torch.bfloat16)
            ops.gemm_tc(x, w, out, bias, ops.EPI_STORE_BF16)
        elif epilogue == "f32":
            out = torch.full((M, N), 7.0, device=DEV)
            ops.gemm_tc(x, w, out, bias, ops.EPI_STORE_F32)
        elif epilogue == "accum":
            base = torch.randn(M, N, device=DEV, generator=g)
            out = base.clone()
            ops.gemm_tc(x, w, out, None, ops.EPI_ACCUM_F32)
            want = want + base.double()
        else:  # rows of w interleaved in blocks of 16 gate, 16 up
            out = torch.full((M, N // 2), 7.0, device=DEV, dtype=torch.bfloat16)
            ops.gemm_tc(x, w, out, None, ops.EPI_SWIGLU_BF16)
            pairs = want.view(M, N // 32, 2, 16)
            want = (torch.nn.functional.silu(pairs[:, :, 0]) * pairs[:, :, 1]).reshape(M, N // 2)
        torch.cuda.synchronize()
        assert ops.gemm_tc_error() == 0
        limit = 1.2e-2 if epilogue in ("bf16", "swiglu") else 2e-5 * max(1.0, math.sqrt(K) / 8)
        error = (out.double() - want).abs().max().item() / (want.abs().max().item() + 1e-6)
        assert error <= limit, (M, N, K, epilogue, bias is not None, error)


@pytest.mark.parametrize("seed", [7, 8])
def test_mixed_steps_of_random_shape_through_both_attention_kernels(seed):
    from torchlet_b200 import ops

    rng = random.Random(seed)
    to = lambda values: torch.tensor(values, dtype=torch.int32, device=DEV)
    for trial in range(40):
        d, nkv, group = rng.choice([64, 128]), rng.choice([1, 2, 4]), rng.choice([1, 2, 3, 5, 7, 8, 16])
        nh, page = nkv * group, rng.choice([8, 16, 32, 64])
        window = rng.choice([None, None, 40, 150, 700])
        n = rng.randint(1, 6)
        before = [rng.choice([0, rng.randint(1, 60), rng.randint(61, 700), rng.randint(701, 2500)]) for _ in range(n)]
        q_lens = [1 if (b > 0 and rng.random() < 0.5) else rng.choice([2, rng.randint(3, 50), rng.randint(51, 400)])
                  for b in before]
        x = kernels.paged_inputs(before, q_lens, nh, nkv, d, page, torch.bfloat16, seed=100 * seed + trial)
        scale = 0.4 / math.sqrt(d)
        want = kernels.plain_attention(x["dense"], before, nh, nkv, window, scale)
        out = torch.full((x["T"], nh * d), float("nan"), device=DEV, dtype=torch.bfloat16)
        decoding = [i for i, q in enumerate(q_lens) if q == 1]
        portions = [i for i, q in enumerate(q_lens) if q > 1]
        merge = None
        if portions:
            rows = ops.attention_tc_rows(group)
            tiles = [(i, start) for i in portions for start in range(0, q_lens[i] * group, rows)]
            merge = ops.attention_tc(x["qkv"], x["pages"], x["table"], x["indptr"], x["before"], to([t[0] for t in tiles]),
                                     to([t[1] for t in tiles]), len(tiles), out, nh, nkv, d, page, window, scale,
                                     splits=rng.choice([1, 1, 2, 3]), token_req=x["token_req"], defer_merge=bool(decoding))
        if decoding:
            ops.attention_mma(x["qkv"], x["pages"], x["table"], x["indptr"], x["before"], to(decoding), None, len(decoding),
                              out, x["T"], nh, nkv, d, page, window, scale, rows16=True,
                              splits=rng.choice([1, 2, 5, 13, 20, 40]), late_wait=bool(portions))
        if merge is not None:
            merge()
        host = out.float().cpu()
        assert ops.attention_tc_error() == 0 and ops.attention_mma_error() == 0
        case = (d, nkv, group, page, window, before, q_lens)
        assert torch.isfinite(host).all(), case
        assert (host - want).abs().max() <= 1.5e-2 * want.abs().max(), case
