"""CPU tests of the oracle itself: it is pinned against vectors produced by the reference's own
kernels (tests/golden/, made by tests/golden/make_golden.py on a GPU), against torch's float8
cast, and against exact integer arithmetic."""
from pathlib import Path

import numpy as np
import pytest
import torch

GOLDEN = sorted((Path(__file__).parent / "golden").glob("ref_sgemm_*.npz"))


def test_golden_files_present():
    assert len(GOLDEN) >= 5


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: p.stem)
def test_sgemm_seq_matches_reference_kernel_output(oracle, path):
    z = np.load(path)
    gen, seed, M, K, N = str(z["gen"]), int(z["seed"]), int(z["M"]), int(z["K"]), int(z["N"])
    A, B = (oracle.gen_randn_f32 if gen == "randn" else oracle.gen_uniform_f32)(M, K, N, seed=seed)
    # the inputs regenerated here are the ones the reference kernels saw
    assert float(A.double().sum()) == float(z["a_checksum"]) and float(B.double().sum()) == float(z["b_checksum"])
    want = torch.from_numpy(z["C"])
    assert torch.equal(oracle.sgemm_seq(A, B), want)                 # bit-exact with the reference kernels
    assert oracle.rel_frobenius(want, oracle.matmul_cpu(A, B)) <= 1e-5


def test_sgemm_seq_exact_on_integers(oracle):
    g = torch.Generator().manual_seed(1)
    A = torch.randint(-8, 9, (37, 53), generator=g).float()
    B = torch.randint(-8, 9, (53, 29), generator=g).float()
    want = (A.long() @ B.long()).float()
    assert torch.equal(oracle.sgemm_seq(A, B), want)
    assert torch.equal(oracle.matmul_f64(A, B).float(), want)


def test_sgemm_seq_order_is_k_ascending_single_accumulator(oracle):
    # a case where the summation order changes the FP32 result: 1e8 + 1 - 1e8
    A = torch.tensor([[1e8, 1.0, -1e8]])
    B = torch.ones(3, 1)
    assert float(oracle.sgemm_seq(A, B)) == 0.0          # (1e8 + 1) rounds to 1e8, then - 1e8
    A2 = torch.tensor([[1e8, -1e8, 1.0]])
    assert float(oracle.sgemm_seq(A2, B)) == 1.0


def test_sgemm_seq_uses_a_fused_multiply_add(oracle):
    # a * b + c with a*b not representable: fused and unfused differ
    a = np.float32(1 + 2 ** -12); b = np.float32(1 + 2 ** -12); c = -np.float32(a * b)
    A = torch.tensor([[1.0, float(a)]]); B = torch.tensor([[float(c)], [float(b)]])   # acc = c, then fma(a, b, acc)
    got = float(oracle.sgemm_seq(A, B))
    assert got == 2.0 ** -24                               # the bits the unfused product rounds away
    

def test_flush_to_zero(oracle):
    A = torch.full((2, 4), 1e-30); B = torch.full((4, 2), 1e-10)
    assert torch.count_nonzero(oracle.sgemm_seq(A, B, ftz=True)) == 0
    assert torch.count_nonzero(oracle.sgemm_seq(A, B, ftz=False)) == 4


def test_empty_k(oracle):
    assert torch.count_nonzero(oracle.sgemm_seq(torch.empty(3, 0), torch.empty(0, 4))) == 0


def test_e4m3_encode_matches_torch_cast(oracle):
    g = torch.Generator().manual_seed(0)
    x = torch.cat([torch.randn(200000, generator=g) * s for s in (1e-3, 1.0, 30.0, 300.0)])
    x = torch.cat([x, torch.tensor([0.0, -0.0, 448.0, 449.0, 464.0, 480.0, 1e9, -1e9, 2.0 ** -9, 2.0 ** -10,
                                    1.5 * 2.0 ** -9, 2.5 * 2.0 ** -9, 2.0 ** -6, 0.0156, 447.9, 432.0, 440.0])])
    want = x.clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(oracle.e4m3_encode(x.numpy()), want)


def test_e4m3_decode_table_matches_torch(oracle):
    t = oracle.e4m3_decode_table()
    want = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()
    assert np.array_equal(np.isnan(t), np.isnan(want))
    assert np.array_equal(t[~np.isnan(t)], want[~np.isnan(want)])
    # every finite value survives encode(decode(.))
    finite = ~np.isnan(t)
    codes = np.arange(256)[finite]
    back = oracle.e4m3_encode(t[finite])
    assert np.array_equal(back[codes != 0x80], codes[codes != 0x80].astype(np.uint8))


def test_mxfp8_recipe(oracle):
    g = torch.Generator().manual_seed(2)
    X = (torch.randn(64, 256, generator=g) * torch.exp(torch.randn(64, 1, generator=g) * 4)).bfloat16()
    X[0, :32] = 0
    q, s = oracle.mxfp8_quantize(X)
    assert q.shape == (64, 256) and s.shape == (64, 8)
    assert int(s[0, 0]) == 0 and int(q[0, :32].max()) == 0          # zero block: byte 0, zero data
    blocks = X.float().view(64, 8, 32)
    amax = blocks.abs().amax(dim=2)
    nz = amax > 0
    # scale = 2^(floor(log2 amax) - 8)
    e = torch.floor(torch.log2(amax[nz])) - 8
    assert torch.equal(s[nz].long() - 127, e.long())
    # scaled magnitudes sit in [256, 512) and are clipped at 448
    dq = oracle.mxfp8_dequantize(q, s)
    scaled = (dq.view(64, 8, 32) / torch.exp2(s.float() - 127)[:, :, None]).abs().amax(dim=2)
    assert float(scaled[nz].min()) >= 256 and float(scaled.max()) <= 448
    # unclipped elements are within half an e4m3 step (2^-4 relative) of the input
    keep = (blocks.abs() / torch.exp2(s.float() - 127)[:, :, None]) <= 448
    rel = ((dq.view(64, 8, 32) - blocks).abs() / blocks.abs().clamp_min(1e-30))[keep & (blocks != 0)]
    big = (blocks.abs() / torch.exp2(s.float() - 127)[:, :, None])[keep & (blocks != 0)] >= 2.0 ** -6
    assert float(rel[big].max()) <= 2.0 ** -4


def test_scale_packing(oracle):
    rows, K = 300, 32 * 10
    s = torch.arange(rows * 10, dtype=torch.int64).remainder(251).to(torch.uint8).view(rows, 10)
    packed = oracle.mxfp8_pack_scales(s, K)
    assert packed.numel() == oracle.mxfp8_scale_bytes(rows, K) == 3 * 3 * 512
    for r, kb in [(0, 0), (31, 3), (32, 0), (127, 9), (128, 4), (299, 9)]:
        assert int(packed[oracle.mxfp8_scale_offset(rows, K, r, kb)]) == int(s[r, kb])
    assert int(packed.sum()) == int(s.long().sum())                   # padding is zero


def test_mxfp8_quantiser_matches_torch_casts_per_block(oracle):
    """Independent pin of the recipe: the same quantisation composed from torch's own float8 casts
    (float8_e8m0fnu for the power-of-two scale, float8_e4m3fn for the data), block by block."""
    g = torch.Generator().manual_seed(11)
    X = (torch.randn(96, 512, generator=g) * torch.exp(torch.randn(96, 1, generator=g) * 5)).bfloat16()
    X[3, 64:96] = 0                                                   # all-zero block
    X[5, :32] = torch.linspace(1.0, 1.99, 32).bfloat16()              # values that clip at 448
    q, s = oracle.mxfp8_quantize(X)
    blocks = X.float().view(96, 16, 32)
    amax = blocks.abs().amax(dim=2)
    nz = amax > 0
    scale = torch.exp2(torch.floor(torch.log2(amax.clamp_min(2.0 ** -126))) - 8)
    scale_byte = scale.to(torch.float8_e8m0fnu).view(torch.uint8)
    assert torch.equal(s[nz], scale_byte[nz])
    assert int(s[~nz].max()) == 0
    back = scale_byte.view(torch.float8_e8m0fnu).float()              # what the scale byte decodes to
    data = (blocks / back[:, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
    keep = nz[:, :, None].expand_as(blocks)
    assert torch.equal(q.view(96, 16, 32)[keep], data[keep])
    assert int(q.view(96, 16, 32)[~keep].max()) == 0
    # and the dequantiser against torch's decode of the same bytes
    dq = oracle.mxfp8_dequantize(q, s).view(96, 16, 32)
    want = q.view(torch.float8_e4m3fn).float().view(96, 16, 32) * s.view(torch.float8_e8m0fnu).float()[:, :, None]
    assert torch.equal(dq[keep], want[keep])
