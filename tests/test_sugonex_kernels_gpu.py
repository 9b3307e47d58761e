"""The kernels that came with the side-by-side layer, the attention over a cached latent and the gated delta rule,
against plain PyTorch float32 restatements of the same operations (tests/cpu_ops.py), in float32 and bfloat16, at
sizes that take the 16-byte paths and sizes that do not."""

import pytest
import torch

from dli_b200.kernels import gemm, ops
from tests import cpu_ops as ref

pytestmark = pytest.mark.gpu

DTYPES = [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)]


def _rand(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g) * scale


def _close(got, want, tol, what=""):
    got, want = got.float().cpu(), want.float()
    err = (got - want).abs().max().item()
    assert err <= tol * max(1.0, want.abs().max().item()), f"{what}: max error {err}"


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("H", [40, 77, 256, 1000, 4096, 8200, 20000])
def test_add_rmsnorm_pair(dtype, tol, H):
    n = 7
    h = _rand(n, H, seed=1) * 3 + 0.5
    a, b = (_rand(n, H, seed=2) * 2 + 1).to(dtype), (_rand(n, H, seed=5) - 0.5).to(dtype)
    w1, w2 = 1 + 0.1 * _rand(H, seed=3), 1 + 0.1 * _rand(H, seed=4)
    for da, db in ((a, b), (a, None), (None, b), (None, None)):
        for two in (True, False):
            for rows in (None, torch.tensor([5, 0, 3], dtype=torch.int32)):
                h_ref, h_dev = h.clone(), h.cuda()
                k = n if rows is None else rows.numel()
                y_ref = [torch.empty(k, H, dtype=dtype) for _ in range(2)]
                y_dev = [torch.empty(k, H, dtype=dtype, device="cuda") for _ in range(2)]
                ref.add_rmsnorm_pair(y_ref[0], y_ref[1] if two else None, h_ref, da, db, w1, w2 if two else None, 1e-5, rows)
                ops.add_rmsnorm_pair(y_dev[0], y_dev[1] if two else None, h_dev, None if da is None else da.cuda(), None if db is None else db.cuda(),
                                     w1.cuda(), w2.cuda() if two else None, 1e-5, None if rows is None else rows.cuda())
                _close(y_dev[0], y_ref[0], tol, "y1")
                if two:
                    _close(y_dev[1], y_ref[1], tol, "y2")
                _close(h_dev, h_ref, 1e-5, "h")


@pytest.mark.parametrize("dtype,tol", DTYPES)
def test_gated_feed_forward_activations(dtype, tol):
    for kind in ops.GLU_ACTIVATIONS:
        for inter, tiled in ((24, False), (37, False), (128, True), (192, False)):
            gu = (_rand(6, 2 * inter, seed=4) * 3).to(dtype)
            want, got = torch.empty(6, inter, dtype=dtype), torch.empty(6, inter, dtype=dtype, device="cuda")
            ref.silu_mul(want, gu, tiled, kind)
            ops.silu_mul(got, gu.cuda(), tiled, kind)
            _close(got, want, tol, f"{kind} {inter}")
    # the same inside the products' epilogues (bfloat16 only): a decode step's few tokens, and a long portion
    if dtype == torch.bfloat16:
        for kind in ops.GLU_ACTIVATIONS:
            for tokens in (3, 700):
                x, wt = (_rand(tokens, 256, seed=6) * 0.5).to(dtype), (_rand(512, 256, seed=7) * 0.1).to(dtype)
                want = ref.skinny_gemm_swiglu(x, wt, kind)
                got = (ops.skinny_gemm_swiglu if tokens <= 8 else ops.dense_gemm_swiglu)(x.cuda(), wt.cuda(), kind)
                _close(got, want, tol, f"{kind} in the epilogue, {tokens} tokens")


def test_scale_softcap():
    x = _rand(5, 1001, seed=1) * 20
    for scale, cap in ((0.5, 15.0), (1.0, 0.0), (2.0, 3.0)):
        want, got = x.clone(), x.cuda()
        ref.scale_softcap(want, scale, cap)
        ops.scale_softcap(got, scale, cap)
        _close(got, want, 1e-6, f"scale {scale} cap {cap}")


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("nh,d,dr,r,rot", [(4, 16, 16, 24, 16), (3, 10, 6, 21, 4), (8, 64, 32, 96, 32), (2, 24, 0, 40, 0), (16, 128, 64, 512, 64)])
@pytest.mark.parametrize("extra", [13, 16])  # columns behind q | down: rows that are and are not 16-byte aligned
def test_latent_prep(dtype, tol, nh, d, dr, r, rot, extra):
    n, page, pages = 9, 8, 5
    row = r + dr
    proj = _rand(n, nh * (d + dr) + row + extra, seed=1).to(dtype)
    w = 1 + 0.2 * _rand(r, seed=2)
    positions = torch.tensor([0, 1, 5, 700, 33, 2, 100000, 7, 64], dtype=torch.int32)
    inv = (1.0 / (10000.0 ** (torch.arange(0, rot, 2).float() / rot))) if rot else None
    slots = torch.tensor([3, 39, 8, 0, 17, 25, 31, 12, 20], dtype=torch.int32)
    for write in (True, False):
        q_ref, q_dev = torch.zeros(n, nh * row, dtype=dtype), torch.zeros(n, nh * row, dtype=dtype, device="cuda")
        k_ref, k_dev = torch.zeros(pages, 1, page, row, dtype=dtype), torch.zeros(pages, 1, page, row, dtype=dtype, device="cuda")
        ref.latent_prep(q_ref, proj, w, 1e-5, positions, inv, slots if write else None, k_ref if write else None, nh, d, dr, r, rot, page)
        ops.latent_prep(q_dev, proj.cuda(), w.cuda(), 1e-5, positions.cuda(), None if inv is None else inv.cuda(), slots.cuda() if write else None,
                        k_dev if write else None, nh, d, dr, r, rot, page)
        _close(q_dev, q_ref, tol, "rotated query parts")
        _close(k_dev, k_ref, tol, "cache rows")


@pytest.mark.parametrize("dtype,tol", DTYPES)
def test_heads_product_into_column_slices(dtype, tol):
    n, heads, d, r, row = 11, 3, 16, 24, 40
    x = _rand(n, heads * (d + 8), seed=1).to(dtype)
    w = (_rand(heads, d, r, seed=2) * 0.3).to(dtype)
    out = torch.full((n, heads * row), 7.0, dtype=dtype, device="cuda")
    gemm.heads_product(x.cuda().view(n, heads, d + 8)[:, :, :d], w.cuda(), out.view(n, heads, row)[:, :, :r])
    want = torch.full((n, heads, row), 7.0)
    want[:, :, :r] = torch.einsum("nhd,hdr->nhr", x.view(n, heads, d + 8)[:, :, :d].float(), w.float())
    _close(out.view(n, heads, row), want, tol, "per-head product")


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("n", [1, 5, 8, 40])  # the engine's own kernel up to 8 tokens, the library's batched product beyond
def test_heads_product_with_gate(dtype, tol, n):
    heads, d, feat, row = 3, 24, 40, 56
    x = _rand(n, heads * row, seed=1).to(dtype)
    w = (_rand(heads, d, feat, seed=2) * 0.3).to(dtype)
    gate = _rand(n, heads * feat + 8, seed=3).to(dtype)
    for g in (None, gate[:, 8:]):
        out = torch.empty(n, heads * feat, dtype=dtype, device="cuda")
        gemm.heads_product(x.cuda().view(n, heads, row)[:, :, 5 : 5 + d], w.cuda(), out.view(n, heads, feat), gate=None if g is None else g.cuda())
        want = torch.einsum("nhd,hdf->nhf", x.view(n, heads, row)[:, :, 5 : 5 + d].float(), w.float())
        if g is not None:
            want = want * torch.sigmoid(g.float()).view(n, heads, feat)
        _close(out.view(n, heads, feat), want, tol, f"{n} tokens, gate {g is not None}")


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,d,dv", [(4, 2, 16, 12), (3, 3, 20, 10), (2, 1, 64, 32), (6, 2, 128, 128), (1, 1, 136, 40), (2, 2, 256, 8), (8, 4, 8, 72), (1, 1, 320, 24), (2, 1, 512, 16)])
def test_delta_rule_scan(dtype, tol, heads, kv_heads, d, dv):
    slots = 4
    lens = [1, 37, 0, 5, 70]  # single tokens, portions beyond one tile of tokens, an empty sequence
    n = sum(lens)
    q_start = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    state_slot = torch.tensor([2, 0, 1, 3, 1], dtype=torch.int32)  # (the empty sequence shares a slot: it touches nothing)
    C = 2 * kv_heads * d + heads * dv
    qkv = _rand(n, C, seed=1).to(dtype)
    u = (_rand(n, 2 * heads + 5, seed=2) * 2).to(dtype)
    dt_bias, a_log = _rand(heads, seed=3) - 1.0, -3.0 + _rand(heads, seed=4)
    state = _rand(slots, heads, dv, d, seed=5) * 0.5
    s_ref, s_dev = state.clone(), state.cuda()
    o_ref, o_dev = torch.zeros(n, heads * dv), torch.zeros(n, heads * dv, device="cuda")
    seq_of = torch.repeat_interleave(torch.arange(len(lens), dtype=torch.int32), torch.tensor(lens))
    ref.delta_rule_scan(o_ref, qkv, u, 3, 3 + heads, dt_bias, a_log, s_ref, seq_of, q_start, state_slot, kv_heads, d, 1e-6)
    ops.delta_rule_scan(o_dev, qkv.cuda(), u.cuda(), 3, 3 + heads, dt_bias.cuda(), a_log.cuda(), s_dev, seq_of.cuda(), q_start.cuda(), state_slot.cuda(),
                        kv_heads, d, 1e-6, max_len=max(lens))
    _close(o_dev, o_ref, 1e-4, "o")  # float32 whatever the inputs' dtype
    _close(s_dev, s_ref, 1e-4, "state")


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("inner,parts", [(48, 4), (70, 5), (512, 2), (4096, 32)])
def test_group_norm_with_the_gate_behind_it(dtype, tol, inner, parts):
    n = 5
    y = _rand(n, inner, seed=1) * 2
    u = _rand(n, inner + 16, seed=2).to(dtype)
    w = 1 + 0.2 * _rand(inner, seed=3)
    for gate_after in (True, False):
        want, got = torch.empty(n, inner, dtype=dtype), torch.empty(n, inner, dtype=dtype, device="cuda")
        ref.gated_group_rmsnorm(want, y, u, 16, w, parts, 1e-5, gate_after)
        ops.gated_group_rmsnorm(got, y.cuda(), u.cuda(), 16, w.cuda(), parts, 1e-5, gate_after)
        _close(got, want, tol, f"gate_after={gate_after}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d", [272, 576, 1000])
def test_attention_on_cuda_cores_beyond_256(dtype, d):
    """One KV head whose rows serve as keys and values, wider than the tensor-core kernels take."""
    n, nh, page, pages = 6, 3, 8, 6
    q = (_rand(n, nh * d, seed=1) * 0.2).to(dtype)
    pool = _rand(pages, 1, page, d, seed=2).to(dtype)
    tables = torch.tensor([[4, 1, 3], [0, 2, 5]], dtype=torch.int32)
    seq_of_token = torch.tensor([0, 0, 0, 1, 1, 1], dtype=torch.int32)
    positions = torch.tensor([3, 17, 23, 0, 9, 20], dtype=torch.int32)
    for window in (None, 6):
        want, got = torch.empty(n, nh * d, dtype=dtype), torch.empty(n, nh * d, dtype=dtype, device="cuda")
        ref.paged_attention_simt(want, q, pool, pool, tables, seq_of_token, positions, nh, 0.3, window)
        dev_pool = pool.cuda()
        ops.paged_attention_simt(got, q.cuda(), dev_pool, dev_pool, tables.cuda(), seq_of_token.cuda(), positions.cuda(), nh, 0.3, window)
        _close(got, want, 2e-5 if dtype == torch.float32 else 2e-2, f"head size {d}, window {window}")
