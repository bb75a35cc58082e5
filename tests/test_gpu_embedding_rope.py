"""Token-embedding gather (bit-exact) + its backward, and rotary, through the C ABI."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import cpu_oracle as O
from tests import tol
from tests.gpu_util import bits, check, make, to_dev
from thot_b200 import abi

pytestmark = pytest.mark.gpu


def test_embedding_golden(golden_dir):
    g = np.load(golden_dir / "embedding.npz")
    table = to_dev(g["table"], torch.float32)
    ids = torch.from_numpy(g["ids"]).cuda()
    out = abi.embedding_fwd(table, ids)
    assert out.shape == (3, 9, 40)
    assert out.cpu().numpy().tobytes() == g["out"].tobytes()
    assert abi.embedding_fwd(table, ids.int()).cpu().numpy().tobytes() == g["out"].tobytes()
    dt = abi.embedding_bwd(to_dev(g["dout"], torch.float32), ids, 64)
    check(dt, g["dtable_f32"], "dtable")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("vocab,D,tokens", [(1, 1, 1), (10, 7, 33), (100, 40, 257), (1000, 1024, 4096), (50, 4100, 9)])
@pytest.mark.parametrize("itype", [torch.int32, torch.int64])
def test_embedding_bit_exact_and_backward(dtype, vocab, D, tokens, itype):
    table, _ = make((vocab, D), vocab + D, dtype, 0.02)
    gen = torch.Generator().manual_seed(tokens)
    ids = torch.randint(0, vocab, (tokens,), generator=gen).to(itype)
    out = abi.embedding_fwd(table, ids.cuda())
    assert torch.equal(out, table[ids.long().cuda()])                 # bit-exact
    host = table.cpu()
    ref, bad = O.embedding(host.view(torch.int16 if dtype == torch.bfloat16 else torch.int32).numpy(), ids.numpy())
    assert bad == -1
    got = out.cpu().view(torch.int16 if dtype == torch.bfloat16 else torch.int32).numpy()
    assert got.tobytes() == ref.tobytes()
    dout, dn = make((tokens, D), tokens + 5, dtype)
    dt = abi.embedding_bwd(dout, ids.cuda(), vocab)
    check(dt, O.embedding_bwd(dn, ids.numpy(), vocab), "dtable")
    assert torch.equal(dt, abi.embedding_bwd(dout, ids.cuda(), vocab))       # deterministic


def test_embedding_bad_ids_do_not_fault():
    table, _ = make((16, 64), 1, torch.float32)
    ids = torch.tensor([3, 16, -2, 5], dtype=torch.int64).cuda()
    status = torch.zeros(2, dtype=torch.int64, device="cuda")
    out = abi.embedding_fwd(table, ids, status)
    assert status[0].item() == 1 and status[1].item() in (1, 2)
    assert float(out[1].abs().sum()) == 0.0 and float(out[2].abs().sum()) == 0.0
    assert torch.equal(out[0], table[3]) and torch.equal(out[3], table[5])
    dt = abi.embedding_bwd(torch.ones(4, 64, device="cuda"), ids, 16)    # bad ids contribute nothing
    assert float(dt.sum()) == 2 * 64


def test_embedding_bad_ids_with_wide_rows():
    """Rows of 1 KiB and more go through the copy-engine gather; a bad id there is a zero row too."""
    table, _ = make((32, 2048), 2, torch.bfloat16)
    ids = torch.tensor([5, -1, 31, 32, 0, 7, 7, 40, 1], dtype=torch.int32).cuda()
    status = torch.zeros(2, dtype=torch.int64, device="cuda")
    out = abi.embedding_fwd(table, ids, status)
    assert status[0].item() == 1
    good = (ids >= 0) & (ids < 32)
    assert torch.equal(out[good], table[ids[good].long()])
    assert float(out[~good].float().abs().sum()) == 0.0
    assert abi.device_status() == 0


def test_config4_embedding_full_size_bit_exact():
    """table[32000,4096] bf16 ~N(0,0.02), int32 ids [32,2048] uniform."""
    torch.manual_seed(0)
    table = (0.02 * torch.randn(32000, 4096)).bfloat16()
    ids = torch.randint(0, 32000, (32, 2048), dtype=torch.int32)
    out = abi.embedding_fwd(table.cuda(), ids.cuda()).cpu()
    ref, bad = O.embedding(table.view(torch.int16).numpy(), ids.numpy())
    assert bad == -1
    assert out.view(torch.int16).numpy().reshape(-1, 4096).tobytes() == ref.tobytes()


def test_config4_embedding_backward_full_size_against_the_oracle():
    """dtable[32000,4096] from dout[65536,4096] bf16 and int32 ids [32,2048]: every table row against the C
    oracle's scatter-add (fp64 sums in ascending token order, rounded once to bf16), one-call and indexed forms."""
    vocab, D, tokens = 32000, 4096, 32 * 2048
    gen = torch.Generator().manual_seed(44)
    ids = torch.randint(0, vocab, (32, 2048), generator=gen, dtype=torch.int32)
    dout = torch.randn(tokens, D, generator=gen).bfloat16()
    got = abi.embedding_bwd(dout.cuda(), ids.cuda(), vocab)
    ref = O.embedding_bwd(dout.float().numpy(), ids.numpy().reshape(-1), vocab)
    check(got, ref, "config 4 dtable")
    counts = np.bincount(ids.numpy().reshape(-1), minlength=vocab)
    assert float(got[torch.from_numpy(counts == 0).cuda()].float().abs().sum()) == 0.0     # unused rows are zero
    index = abi.embedding_index(ids.cuda(), vocab)
    assert torch.equal(abi.embedding_bwd_indexed(dout.cuda(), index, vocab), got)
    assert abi.device_status() == 0


def test_rope_table_matches_oracle():
    for S, hd, theta in [(2048, 128, 10000.0), (17, 64, 500000.0), (5, 2, 10000.0), (3, 1024, 10000.0)]:
        cs = abi.rope_table(S, hd, theta).cpu().numpy()
        ref = O.rope_table(S, hd, theta)
        # same formula, fp64 cos/sin rounded once: equal up to a last-bit double-rounding case
        np.testing.assert_allclose(cs, ref, rtol=0, atol=6e-8)
    pos = torch.tensor([7, 0, 2047, 3], dtype=torch.int32)
    cs = abi.rope_table(4, 128, 10000.0, positions=pos.cuda()).cpu().numpy()
    np.testing.assert_allclose(cs, O.rope_table(4, 128, 10000.0, positions=pos.numpy()), rtol=0, atol=6e-8)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,S,H,hd", [(1, 1, 1, 2), (2, 5, 3, 6), (2, 33, 4, 64), (3, 17, 8, 128), (1, 9, 2, 256)])
def test_rope_apply_and_inverse(dtype, B, S, H, hd):
    x, xn = make((B, S, H, hd), B * 1000 + S + hd, dtype)
    cs = abi.rope_table(S, hd)
    csn = cs.cpu().numpy()
    y = abi.rope_apply(x, cs)
    check(y, O.rope_apply(xn, csn), "rope fwd")
    dy, dyn = make((B, S, H, hd), 77, dtype)
    check(abi.rope_apply(dy, cs, inverse=True), O.rope_apply(dyn, csn, inverse=True), "rope bwd")
    if dtype == torch.float32:     # rotation then inverse rotation restores the input
        back = abi.rope_apply(y, cs, inverse=True)
        np.testing.assert_allclose(back.cpu().numpy(), xn, atol=2e-6)


def test_config4_rope_full_size_sampled():
    """q,k[32,2048,32,128] bf16, theta=10000, positions 0..2047."""
    B, S, H, hd = 32, 2048, 32, 128
    gen = torch.Generator(device="cuda").manual_seed(4)
    cs = abi.rope_table(S, hd)
    csn = cs.cpu().numpy()
    for seed_shift in (0, 1):      # q then k
        x = torch.randn(B, S, H, hd, device="cuda", generator=gen).bfloat16()
        y = abi.rope_apply(x, cs)
        for b, s0 in ((0, 0), (13, 1000), (31, 2040)):
            xs = x[b:b + 1, s0:s0 + 8].float().cpu().numpy()
            ref = O.rope_apply(xs, csn[s0:s0 + 8])
            check(y[b:b + 1, s0:s0 + 8], ref, f"rope sample b={b} s={s0}")
        # a rotation preserves each pair's norm: whole-tensor checksum in fp32
        n_in = x.float().pow(2).sum(dtype=torch.float64)
        n_out = y.float().pow(2).sum(dtype=torch.float64)
        assert abs(float(n_out / n_in) - 1.0) < 1e-4


@pytest.mark.parametrize("dtype,D", [(torch.float32, 256), (torch.bfloat16, 4096)])
def test_embedding_bwd_with_one_id_used_by_most_tokens(dtype, D):
    """A padding-like id that most tokens share goes through the long-run kernel (columns spread over
    many warps); the sums keep the ascending-token order, so the result equals the oracle's."""
    vocab, tokens = 300, 6000
    gen = torch.Generator().manual_seed(5)
    ids = torch.randint(0, vocab, (tokens,), generator=gen)
    ids[torch.rand(tokens, generator=gen) < 0.7] = 17          # ~4200 tokens share id 17
    ids[::5][:1200] = 250                                       # and a second run just above the threshold
    dout, dn = make((tokens, D), 6, dtype)
    got = abi.embedding_bwd(dout, ids.cuda(), vocab)
    ref = O.embedding_bwd(dn, ids.numpy(), vocab)
    n17 = int((ids == 17).sum())
    assert n17 > 1024 and int((ids == 250).sum()) > 1024
    if dtype == torch.float32:
        tol.long_sum_close(got.cpu().numpy(), ref, n17)
    else:
        # bf16 output of an fp32 sum of n terms: 2 bf16 ulp, and the fp32 sum's own error where it cancels
        np.testing.assert_allclose(got.float().cpu().numpy(), ref, rtol=2.0 ** -7, atol=1e-5 * np.sqrt(n17))
    again = abi.embedding_bwd(dout, ids.cuda(), vocab)
    assert torch.equal(got, again)                              # no atomics on the data: bit-identical reruns


def test_embedding_backward_from_a_prebuilt_index_equals_the_one_call_form():
    """nb2_embedding_index + nb2_embedding_bwd_indexed: same bits as nb2_embedding_bwd, and one index serves
    several backward calls (skewed ids included, so the long-run list is rebuilt per call)."""
    vocab, tokens, D = 500, 9000, 512
    gen = torch.Generator().manual_seed(21)
    ids = torch.randint(0, vocab, (tokens,), generator=gen, dtype=torch.int32)
    ids[::3] = 7                                               # 3000 tokens on one row: the long-run kernel
    idc = ids.cuda()
    index = abi.embedding_index(idc, vocab)
    for seed in (1, 2):
        dout, _ = make((tokens, D), seed, torch.bfloat16)
        assert torch.equal(abi.embedding_bwd_indexed(dout, index, vocab), abi.embedding_bwd(dout, idc, vocab))
    L = abi.lib()
    assert L.nb2_embedding_bwd_indexed(None, None, 4, 8, 16, 0, None, 0, None) == -1            # NULL
    small = torch.empty(64, dtype=torch.uint8, device="cuda")
    dt = torch.empty(vocab, D, device="cuda")
    do = torch.empty(tokens, D, device="cuda")
    import ctypes
    P = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    assert L.nb2_embedding_bwd_indexed(P(do), P(dt), tokens, vocab, D, 0, P(small), 64, None) == -5   # workspace too small
