"""The kernels of the sandwich layers, the sink attention and the state-space mixer against plain PyTorch
float32 restatements of the same operations (tests/cpu_ops.py), in float32 and bfloat16."""

import math

import pytest
import torch

from dli_b200.kernels import ops
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
@pytest.mark.parametrize("H", [40, 77, 256, 1000, 4096, 8200])
def test_post_add_layernorm(dtype, tol, H):
    n = 7
    h = _rand(n, H, seed=1) * 3 + 0.5
    a = (_rand(n, H, seed=2) * 2 + 1).to(dtype)
    w1, w2 = 1 + 0.1 * _rand(H, seed=3), 1 + 0.1 * _rand(H, seed=4)
    for use_a in (True, False):
        for rows in (None, torch.tensor([5, 0, 3], dtype=torch.int32)):
            h_ref, h_dev = h.clone(), h.cuda()
            k = n if rows is None else rows.numel()
            y_ref, y_dev = torch.empty(k, H, dtype=dtype), torch.empty(k, H, dtype=dtype, device="cuda")
            ref.post_add_layernorm(y_ref, h_ref, a if use_a else None, w1 if use_a else None, w2, 1e-5, 1e-6, rows)
            ops.post_add_layernorm(y_dev, h_dev, a.cuda() if use_a else None, w1.cuda() if use_a else None, w2.cuda(), 1e-5, 1e-6,
                                   None if rows is None else rows.cuda())
            _close(y_dev, y_ref, tol, "y")
            _close(h_dev, h_ref, 1e-5, "h")
    # the addition alone
    h_ref, h_dev = h.clone(), h.cuda()
    ref.post_add_layernorm(None, h_ref, a, w1, None, 1e-5, 0.0)
    ops.post_add_layernorm(None, h_dev, a.cuda(), w1.cuda(), None, 1e-5, 0.0)
    _close(h_dev, h_ref, 1e-5, "h alone")


@pytest.mark.parametrize("dtype,tol", DTYPES)
def test_stream_reinject_and_activation(dtype, tol):
    n, H, V = 5, 72, 33
    h = _rand(n, H, seed=1)
    table = _rand(V, H, seed=2).to(dtype)
    ids = torch.tensor([3, 32, 0, 7, 7], dtype=torch.int32)
    vec = _rand(H, seed=3)
    for t, v in ((table, vec), (None, vec), (table, None)):
        h_ref, h_dev = h.clone(), h.cuda()
        ref.stream_reinject(h_ref, t, ids, v)
        ops.stream_reinject(h_dev, None if t is None else t.cuda(), ids.cuda() if t is not None else None, None if v is None else v.cuda())
        _close(h_dev, h_ref, 1e-6)
    for kind in ops.ACTIVATIONS:
        for cols in (24, 37):
            x = (_rand(6, cols, seed=4) * 3).to(dtype)
            want = ref.activation(x.clone(), kind)
            got = ops.activation(x.cuda(), kind)
            _close(got, want, tol, kind)


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("nh,nkv,d,rot,normed,from_keys", [(4, 2, 16, 16, True, True), (3, 1, 32, 8, True, True), (8, 8, 64, 0, False, False),
                                                            (6, 2, 48, 48, True, False), (16, 2, 128, 64, True, True)])
@pytest.mark.parametrize("extra", [13, 16])  # columns behind q | k (| v): rows that are and are not 16-byte aligned
def test_qk_norm_rotary_store(dtype, tol, nh, nkv, d, rot, normed, from_keys, extra):
    n, page, pages = 9, 8, 5
    cols = (nh + (1 if from_keys else 2) * nkv) * d + extra
    proj = _rand(n, cols, seed=1).to(dtype)
    wq, wk = (1 + 0.2 * _rand(nh * d, seed=2), 1 + 0.2 * _rand(nkv * d, seed=3)) if normed else (None, None)
    positions = torch.tensor([0, 1, 2, 700, 701, 5, 6, 7, 8], dtype=torch.int32)
    inv = (1.0 / (10000.0 ** (torch.arange(0, rot, 2).float() / rot)) / 4.0) if rot else None
    slots = torch.randperm(page * pages, generator=torch.Generator().manual_seed(5))[:n].to(torch.int32)
    kp_ref, vp_ref = torch.zeros(pages, nkv, page, d, dtype=dtype), torch.zeros(pages, nkv, page, d, dtype=dtype)
    kp, vp = kp_ref.cuda(), vp_ref.cuda()
    q_ref = ref.qk_norm_rotary_store(proj, wq, wk, 1e-6, positions, inv, slots, kp_ref, vp_ref, nh, nkv, d, rot, page, True, from_keys)
    q = ops.qk_norm_rotary_store(proj.cuda(), None if wq is None else wq.cuda(), None if wk is None else wk.cuda(), 1e-6, positions.cuda(),
                                 None if inv is None else inv.cuda(), slots.cuda(), kp, vp, nh, nkv, d, rot, page, True, from_keys)
    _close(q, q_ref, tol, "q"), _close(kp, kp_ref, tol, "k"), _close(vp, vp_ref, 0.0, "v")
    # a step that reads another step's cache writes nothing
    kp2 = torch.zeros_like(kp)
    q2 = ops.qk_norm_rotary_store(proj.cuda(), None if wq is None else wq.cuda(), None if wk is None else wk.cuda(), 1e-6, positions.cuda(),
                                  None if inv is None else inv.cuda(), None, None, None, nh, nkv, d, rot, page, False, from_keys)
    assert torch.equal(q2, q) and not kp2.any()


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("width,lo", [(100, 50), (104, 48)])
def test_sigmoid_gate(dtype, tol, width, lo):
    out = _rand(6, 40, seed=1).to(dtype)
    wide = (_rand(6, width, seed=2) * 4).to(dtype)
    want = out.clone()
    ref.sigmoid_gate(want, wide[:, lo : lo + 40])
    got = out.cuda()
    ops.sigmoid_gate(got, wide.cuda()[:, lo : lo + 40])
    _close(got, want, tol)


def _batch(q_lens):
    q_start = [0]
    for q in q_lens:
        q_start.append(q_start[-1] + q)
    seq_of = [s for s, q in enumerate(q_lens) for _ in range(q)]
    return torch.tensor(q_start, dtype=torch.int32), torch.tensor(seq_of, dtype=torch.int32)


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("taps", [1, 2, 4])
@pytest.mark.parametrize("C,col0", [(150, 11), (152, 8), (2304, 16)])
@pytest.mark.parametrize("q_lens", [[1, 5, 2, 1], [1, 70, 2, 13]], ids=["few_tokens", "portions"])  # portions take the kernel with a window in registers
def test_causal_conv_and_its_state(dtype, tol, taps, C, col0, q_lens):
    slots = 6
    q_start, seq_of = _batch(q_lens)
    n = int(q_start[-1])
    slot = torch.tensor([4, 0, 5, 2], dtype=torch.int32)
    u = _rand(n, col0 + C + (3 if C % 8 else 8), seed=1).to(dtype)
    w, b = _rand(taps, C, seed=2), _rand(C, seed=3)
    state = _rand(slots, taps - 1, C, seed=4).to(dtype)
    out_ref, out = torch.empty(n, C, dtype=dtype), torch.empty(n, C, dtype=dtype, device="cuda")
    st_ref, st = state.clone(), state.cuda()
    ref.causal_conv_silu(out_ref, u, col0, w, b, st_ref, seq_of, q_start, slot)
    ops.causal_conv_silu(out, u.cuda(), col0, w.cuda(), b.cuda(), st, seq_of.cuda(), q_start.cuda(), slot.cuda())
    _close(out, out_ref, tol)
    if taps > 1:
        ref.conv_state_update(st_ref, u, col0, q_start, slot)
        ops.conv_state_update(st, u.cuda(), col0, q_start.cuda(), slot.cuda())
        _close(st, st_ref, 0.0, "state")


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("heads,P,N,groups", [(6, 48, 32, 2), (4, 64, 128, 1), (3, 20, 10, 3), (2, 96, 256, 2), (8, 8, 64, 4), (1, 5, 33, 1), (160, 40, 24, 8), (2, 16, 320, 1), (1, 8, 512, 1)])
def test_ssm_scan(dtype, tol, heads, P, N, groups):
    q_lens = [1, 77, 2, 32]
    q_start, _ = _batch(q_lens)
    n = int(q_start[-1])
    slot = torch.tensor([3, 1, 0, 4], dtype=torch.int32)
    inner = heads * P
    xbc = _rand(n, inner + 2 * groups * N, seed=1).to(dtype)
    dt_col = 5
    u = _rand(n, dt_col + heads + 2, seed=2).to(dtype)
    dt_bias, a_log, d_skip = _rand(heads, seed=3), _rand(heads, seed=4) * 0.5, _rand(heads, seed=5)
    state = _rand(5, heads, P, N, seed=6)
    y_ref, y = torch.zeros(n, inner), torch.zeros(n, inner, device="cuda")
    st_ref, st = state.clone(), state.cuda()
    ref.ssm_scan(y_ref, xbc, u, dt_col, dt_bias, a_log, d_skip, st_ref, q_start, slot, groups)
    ops.ssm_scan(y, xbc.cuda(), u.cuda(), dt_col, dt_bias.cuda(), a_log.cuda(), d_skip.cuda(), st, q_start.cuda(), slot.cuda(), groups)
    _close(y, y_ref, 1e-4, "y"), _close(st, st_ref, 1e-4, "state")
    # the launch for steps of single tokens (nothing fetched ahead) computes the same
    y2, st2 = torch.zeros(n, inner, device="cuda"), state.cuda()
    ops.ssm_scan(y2, xbc.cuda(), u.cuda(), dt_col, dt_bias.cuda(), a_log.cuda(), d_skip.cuda(), st2, q_start.cuda(), slot.cuda(), groups, max_len=1)
    _close(y2, y_ref, 1e-4, "y, no prefetch"), _close(st2, st_ref, 1e-4, "state, no prefetch")
    assert torch.equal(st[2].cpu(), state[2]), "a slot of no sequence was touched"


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("inner,parts", [(288, 2), (64, 1), (120, 5), (90, 3), (4096, 8), (16384, 1)])
def test_gated_group_rmsnorm(dtype, tol, inner, parts):
    n, z_col = 5, (3 if inner == 90 else 8)
    y = _rand(n, inner, seed=1) * 2
    u = _rand(n, z_col + inner + (4 if inner == 90 else 8), seed=2).to(dtype)
    w = 1 + 0.1 * _rand(inner, seed=3)
    out_ref, out = torch.empty(n, inner, dtype=dtype), torch.empty(n, inner, dtype=dtype, device="cuda")
    ref.gated_group_rmsnorm(out_ref, y, u, z_col, w, parts, 1e-6)
    ops.gated_group_rmsnorm(out, y.cuda(), u.cuda(), z_col, w.cuda(), parts, 1e-6)
    _close(out, out_ref, tol)


def _attention_case(dtype, nh, nkv, d, page, q_lens, kv_lens, seed=0):
    """A batch for the attention kernels: single-token sequences first; returns CPU tensors."""
    g = torch.Generator().manual_seed(seed)
    S = len(q_lens)
    width = max(-(-k // page) for k in kv_lens)
    pages = sum(-(-k // page) for k in kv_lens) + 2
    perm = torch.randperm(pages - 1, generator=g) + 1
    tables = torch.full((S, width), -1, dtype=torch.int32)
    at = 0
    for s, k in enumerate(kv_lens):
        cnt = -(-k // page)
        tables[s, :cnt] = perm[at : at + cnt].to(torch.int32)
        at += cnt
    q_start, seq_of = _batch(q_lens)
    n = int(q_start[-1])
    positions = torch.cat([torch.arange(k - q, k) for q, k in zip(q_lens, kv_lens)]).to(torch.int32)
    qkv = (torch.randn(n, nh * d, generator=g) * 1.5).to(dtype)
    kp = torch.randn(pages, nkv, page, d, generator=g).to(dtype)
    vp = torch.randn(pages, nkv, page, d, generator=g).to(dtype)
    return dict(qkv=qkv, kp=kp, vp=vp, tables=tables, q_start=q_start, seq_of=seq_of, positions=positions,
                kv_len=torch.tensor(kv_lens, dtype=torch.int32), n=n)


@pytest.mark.parametrize("sink", [0.0, 1.5, None])
def test_sink_in_the_float32_attention(sink):
    nh, nkv, d, page = 4, 2, 24, 8
    c = _attention_case(torch.float32, nh, nkv, d, page, [1, 1, 19], [40, 1, 19])
    want = torch.empty(c["n"], nh * d)
    ref.paged_attention_simt(want, c["qkv"], c["kp"], c["vp"], c["tables"], c["seq_of"], c["positions"], nh, 0.3, None, sink)
    got = torch.empty(c["n"], nh * d, device="cuda")
    ops.paged_attention_simt(got, c["qkv"].cuda(), c["kp"].cuda(), c["vp"].cuda(), c["tables"].cuda(), c["seq_of"].cuda(),
                             c["positions"].cuda(), nh, 0.3, None, sink)
    _close(got, want, 1e-5)
    if sink is not None:  # the sink takes mass: a token that sees one key does not return that key's value unchanged
        row = c["q_start"][1]
        assert (got[row].cpu() - c["vp"][c["tables"][1, 0], :, 0].repeat_interleave(nh // nkv, 0).reshape(-1)).abs().max() > 1e-3


@pytest.mark.parametrize("d,page", [(64, 16), (128, 16), (32, 16), (48, 8)])
@pytest.mark.parametrize("sink", [0.0, -2.0])
def test_sink_in_the_bfloat16_attention_kernels(d, page, sink):
    """Prompt portions and single tokens through the tensor-core kernels the engine would choose, with and without
    split keys, against the plain restatement."""
    nh, nkv = 8, 2
    c = _attention_case(torch.bfloat16, nh, nkv, d, page, [1, 1, 1, 150, 3], [1, 300, 77, 150, 203], seed=3)
    want = torch.empty(c["n"], nh * d, dtype=torch.bfloat16)
    scale = 1.0 / math.sqrt(d)
    ref.paged_attention_simt(want, c["qkv"], c["kp"], c["vp"], c["tables"], c["seq_of"], c["positions"], nh, scale, None, sink)
    dev = {k: v.cuda() for k, v in c.items() if isinstance(v, torch.Tensor)}
    singles, total = 3, 5
    for splits in (1, 2, 4):
        got = torch.zeros(c["n"], nh * d, dtype=torch.bfloat16, device="cuda")
        scratch = None
        if splits > 1:
            scratch = (torch.empty(singles * nh * splits * d, device="cuda"), torch.empty(singles * nh * splits * 2, device="cuda"))
        if ops.decode_tma_supported(d, page):
            ops.paged_decode_tma(got, dev["qkv"], dev["kp"], dev["vp"], dev["tables"], dev["q_start"], dev["kv_len"], 0, singles, 0, nh, scale,
                                 None, splits, scratch, 300, sink=sink)
        else:
            ops.paged_attention_mma(got, dev["qkv"], dev["kp"], dev["vp"], dev["tables"], dev["q_start"], dev["kv_len"], 0, singles, 1, 0, nh,
                                    scale, None, splits, scratch, sink=sink)
        if ops.prefill_tc_supported(d, page):
            for tiles in (1, 2) if d == 64 else (0,):
                ops.paged_prefill_tc(got, dev["qkv"], dev["kp"], dev["vp"], dev["tables"], dev["q_start"], dev["kv_len"], singles, total - singles,
                                     150, nh, scale, None, tiles, sink=sink)
                _close(got, want, 3e-2, f"splits {splits} tiles {tiles}")
        else:
            ops.paged_attention_mma(got, dev["qkv"], dev["kp"], dev["vp"], dev["tables"], dev["q_start"], dev["kv_len"], singles, total - singles,
                                    150, singles, nh, scale, None, sink=sink)
            _close(got, want, 3e-2, f"splits {splits}")
    assert ops.device_wait_errors() == {}


@pytest.mark.parametrize("kind", ["relu2", "gelu_tanh", "silu"])
@pytest.mark.parametrize("tokens,K,features", [(1, 256, 384), (5, 2048, 8192), (8, 96, 200)])
def test_decode_product_with_the_activation_in_its_epilogue(kind, tokens, K, features):
    """Equal to the plain product (rounded to bfloat16) followed by the activation kernel, bit for bit up to the
    product's own summation order."""
    x = (_rand(tokens, K, seed=1)).to(torch.bfloat16)
    w = (_rand(features, K, seed=2) / K**0.5).to(torch.bfloat16)
    want = ref.skinny_gemm_act(x, w, kind)
    got = ops.skinny_gemm_act(x.cuda(), w.cuda(), kind)
    _close(got, want, 2e-2, kind)
    two_steps = ops.activation(ops.skinny_gemm(x.cuda(), w.cuda()), kind)
    assert (got.float() - two_steps.float()).abs().max().item() <= 2e-2 * max(1.0, want.float().abs().max().item())


@pytest.mark.parametrize("kind", ["relu2", "gelu_tanh", "silu"])
@pytest.mark.parametrize("tokens,K,features", [(700, 256, 384), (1024, 512, 1032)])
def test_long_portion_product_with_the_activation_in_its_epilogue(kind, tokens, K, features):
    x = (_rand(tokens, K, seed=1)).to(torch.bfloat16)
    w = (_rand(features, K, seed=2) / K**0.5).to(torch.bfloat16)
    want = ref.dense_gemm_act(x, w, kind)
    got = ops.dense_gemm_act(x.cuda(), w.cuda(), kind)
    _close(got, want, 2e-2, kind)
    assert ops.dense_gemm_error() == 0
