"""Fused attention (fml_attention_fwd / fml_attention_bwd) against the oracle's matMul / scaleMatrix / softmaxMatrix
chain (singleHeadAttentionLayer.dart:77-86), per (sequence, head)."""
import ctypes as C
import math

import numpy as np
import pytest

from tests.gpu_util import rel

pytestmark = pytest.mark.gpu


def w64(a):
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32), dtype=np.float64)


def trunc_tf32(x):
    """What the tensor core does to an fp32 operand: the low 13 mantissa bits are dropped (measured on the device: a
    float64 product of operands cut this way reproduces a TF32 product to 3e-7)."""
    b = np.ascontiguousarray(x, np.float32).view(np.uint32) & np.uint32(0xFFFFE000)
    return b.view(np.float32).astype(np.float64)


def round_tf32(x):
    """Round to nearest TF32, ties away from zero: what the kernels do to the operands they build on chip."""
    b = (np.ascontiguousarray(x, np.float32).view(np.uint32) + np.uint32(0x1000)) & np.uint32(0xFFFFE000)
    return b.view(np.float32).astype(np.float64)


def emulate_forward(Q, K, V, scale, causal, lazy=True):
    """The forward kernel's arithmetic in float64 with the TF32 operand handling made explicit: per block of 128
    queries, key blocks of 128; S = trunc(Q).trunc(K)^T, P~ = round(2^(k S - m)) unnormalised against the row's exponent
    reference m; row sum over the ROUNDED P~, O = P~.trunc(V) / l.  Returns O and lse = m + log2 l.  `lazy`: the kernel for
    sequences up to 512 moves m only when a block's maximum exceeds it by more than 2^8 (the accumulated output and row sum
    are rescaled then); the kernel for longer sequences follows the running maximum block by block."""
    S_len = Q.shape[0]
    k2 = np.float32(scale) * np.float32(1.4426950408889634)
    Qt, Kt, Vt = trunc_tf32(Q), trunc_tf32(K), trunc_tf32(V)
    O, lse = np.zeros((S_len, 64)), np.zeros(S_len)
    for q0 in range(0, S_len, 128):
        m = np.full(128, -np.inf)
        l, o = np.zeros(128), np.zeros((128, 64))
        n_kv = q0 // 128 + 1 if causal else S_len // 128
        for j in range(n_kv):
            s = Qt[q0:q0 + 128] @ Kt[j * 128:(j + 1) * 128].T
            if causal and j == q0 // 128:
                s = np.where(np.tril(np.ones((128, 128), bool)), s, -np.inf)
            bm = s.max(1) * k2
            m_new = np.where(bm > m + 8.0, bm, m) if lazy else np.maximum(m, bm)
            alpha = np.where(m_new > m, np.exp2(m - m_new), 1.0)
            pt = round_tf32(np.exp2(s * k2 - m_new[:, None]).astype(np.float32))
            o = o * alpha[:, None] + pt @ Vt[j * 128:(j + 1) * 128]
            l = l * alpha + pt.sum(1)
            m = m_new
        O[q0:q0 + 128] = o / l[:, None]
        lse[q0:q0 + 128] = m + np.log2(l)
    return O, lse


def emulate_backward(Q, K, V, dO, O_dev, lse_dev, scale, causal):
    """The two backward kernels given THEIR inputs (the forward's O and lse as the device produced them): S and dP from
    truncated operands, P = 2^(k S - lse), D = rowsum(dO * O), dS = scale P (dP - D); P and dS rounded to TF32, then
    dQ = dS.trunc(K), dK = dS^T.trunc(Q), dV = P^T.trunc(dO).  Each output is ONE product away from the elementwise
    stage, so agreement here bounds every product of the backward pass on the device's own intermediates."""
    S_len = Q.shape[0]
    k2 = np.float32(scale) * np.float32(1.4426950408889634)
    Qt, Kt, Vt, dOt = trunc_tf32(Q), trunc_tf32(K), trunc_tf32(V), trunc_tf32(dO)
    s = Qt @ Kt.T
    P = np.exp2(s * k2 - lse_dev[:, None].astype(np.float64))
    if causal:
        P = np.where(np.tril(np.ones((S_len, S_len), bool)), P, 0.0)
    D = (dO.astype(np.float64) * O_dev.astype(np.float64)).sum(1, keepdims=True)
    dS = round_tf32((P * (dOt @ Vt.T - D) * scale).astype(np.float32))
    Pr = round_tf32(P.astype(np.float32))
    return dS @ Kt, dS.T @ Qt, Pr.T @ dOt


def attention_desc(ctx, qkv, out, lse, Bn, S, H, causal, scale):
    from flutter_ml_b200 import _lib
    d = _lib.AttentionDesc()
    dm = H * 64
    d.n_seq, d.seq_len, d.heads, d.d_head = Bn, S, H, 64
    d.q, d.k, d.v = qkv.ptr, qkv.ptr + 4 * dm, qkv.ptr + 8 * dm
    d.ld_qkv, d.out, d.ld_out = 3 * dm, out.ptr, dm
    d.lse = lse.ptr if lse is not None else None
    d.scale, d.causal = scale, int(causal)
    return d


@pytest.mark.parametrize("S,causal", [(128, False), (128, True), (384, True), (512, True), (256, False), (1024, True)])
def test_fused_attention_forward(orc, S, causal):
    from flutter_ml_b200 import _lib
    ctx = _lib.Context(precision=_lib.PREC_TF32)
    Bn, H, dk = 2, 3, 64
    dm = H * dk
    rng = np.random.default_rng(S + causal)
    qkv = rng.standard_normal((Bn * S, 3 * dm)).astype(np.float32)
    scale = 1 / math.sqrt(dk)
    dq, out, lse = ctx.upload(qkv), ctx.empty(Bn * S, dm), ctx.empty(Bn * H * S)
    d = attention_desc(ctx, dq, out, lse, Bn, S, H, causal, scale)
    ctx.check(ctx.lib.fml_attention_fwd(ctx.h, C.byref(d)))
    assert ctx.device_status() == 0
    got, got_lse = out.numpy(), lse.numpy().reshape(Bn, H, S)
    ops = orc.Ops(omp=True)
    for b in range(Bn):
        for h in range(H):
            rows = slice(b * S, (b + 1) * S)
            Q, K, V = (w64(qkv[rows, i * dm + h * dk:i * dm + (h + 1) * dk]) for i in range(3))
            s_ref = ops.matmul_fwd(Q, np.ascontiguousarray(K.T)) * scale
            p_ref = ops.softmax_fwd(s_ref, S if causal else 0)
            o_ref = ops.matmul_fwd(p_ref, V)
            # Against exact float64 arithmetic: a chain of two products whose fp32 operands the tensor core truncates
            # (each truncated operand biases a product low by about 3.5e-4, and the biases of a chain add up).
            assert rel(got[rows, h * dk:(h + 1) * dk], o_ref) <= 2e-3
            # Against the same chain with that operand handling made explicit: the kernel itself adds nothing beyond
            # fp32 accumulation and the hardware exponential.
            Q32, K32, V32 = (qkv[rows, i * dm + h * dk:i * dm + (h + 1) * dk] for i in range(3))
            o_emu, lse_emu = emulate_forward(Q32, K32, V32, scale, causal, lazy=S <= 512)
            assert rel(got[rows, h * dk:(h + 1) * dk], o_emu) <= 2e-4, rel(got[rows, h * dk:(h + 1) * dk], o_emu)
            assert np.max(np.abs(got_lse[b, h] - lse_emu)) <= 1e-4
            masked = np.where(np.tril(np.ones((S, S), bool)) | (not causal), s_ref, -np.inf)
            lse_ref = (np.log(np.exp(masked - masked.max(1, keepdims=True)).sum(1)) + masked.max(1)) / math.log(2)
            assert np.max(np.abs(got_lse[b, h] - lse_ref)) <= 2e-2
    ctx.close()


@pytest.mark.parametrize("S,causal", [(256, False), (512, True), (512, False)])
def test_fused_attention_forward_moves_the_exponent_reference(S, causal):
    """Keys whose magnitude changes from block to block (x1, x3.2, x1/3, x4.5): in many rows, but not in all rows of a warp, a
    later block's maximum exceeds the exponent reference by more than 2^8, so the accumulator in tensor memory is rescaled in
    the middle of an item (random data of one magnitude never gets there).  Output and row statistics against the float64
    emulation of the kernel's rule, and against exact softmax attention; the moved rows are counted."""
    from flutter_ml_b200 import _lib
    ctx = _lib.Context(precision=_lib.PREC_TF32)
    Bn, H, dk = 1, 2, 64
    dm = H * dk
    rng = np.random.default_rng(7 * S + causal)
    qkv = rng.standard_normal((Bn * S, 3 * dm)).astype(np.float32)
    gain = np.array([1.0, 3.2, 1.0 / 3.0, 4.5], np.float32)
    for j in range(S // 128):
        qkv[j * 128:(j + 1) * 128, dm:2 * dm] *= gain[j]
    scale = 1 / math.sqrt(dk)
    dq, out, lse = ctx.upload(qkv), ctx.empty(Bn * S, dm), ctx.empty(Bn * H * S)
    d = attention_desc(ctx, dq, out, lse, Bn, S, H, causal, scale)
    ctx.check(ctx.lib.fml_attention_fwd(ctx.h, C.byref(d)))
    assert ctx.device_status() == 0
    got, got_lse = out.numpy(), lse.numpy().reshape(Bn, H, S)
    k2 = scale * 1.4426950408889634
    for h in range(H):
        Q32, K32, V32 = (qkv[:, i * dm + h * dk:i * dm + (h + 1) * dk] for i in range(3))
        # how many rows move their reference after the first block, and how many keep it although a neighbour moves
        s = trunc_tf32(Q32) @ trunc_tf32(K32).T * k2
        moved = np.zeros(S, bool)
        for q0 in range(0, S, 128):
            m = np.full(128, -np.inf)
            for j in range(q0 // 128 + 1 if causal else S // 128):
                blk = s[q0:q0 + 128, j * 128:(j + 1) * 128]
                if causal and j == q0 // 128:
                    blk = np.where(np.tril(np.ones((128, 128), bool)), blk, -np.inf)
                mv = blk.max(1) > m + 8.0
                if j > 0:
                    moved[q0:q0 + 128] |= mv
                m = np.where(mv, blk.max(1), m)
        per_warp = moved.reshape(-1, 32)
        mixed = int(((per_warp.sum(1) > 0) & (per_warp.sum(1) < 32)).sum())
        print(f"S {S} causal {causal} head {h}: rows that move the reference after block 0: {int(moved.sum())} of {S}, "
              f"warps with both kinds of rows: {mixed}")
        assert moved.sum() > S // 8 and mixed > 0
        o_emu, lse_emu = emulate_forward(Q32, K32, V32, scale, causal, lazy=True)
        assert rel(got[:, h * dk:(h + 1) * dk], o_emu) <= 2e-4, rel(got[:, h * dk:(h + 1) * dk], o_emu)
        assert np.max(np.abs(got_lse[0, h] - lse_emu)) <= 2e-4
        sc = w64(Q32) @ w64(K32).T * scale
        if causal:
            sc = np.where(np.tril(np.ones((S, S), bool)), sc, -np.inf)
        pr = np.exp(sc - sc.max(1, keepdims=True))
        o_ref = (pr / pr.sum(1, keepdims=True)) @ w64(V32)
        assert rel(got[:, h * dk:(h + 1) * dk], o_ref) <= 5e-3    # sharply peaked rows: the truncation of one dominant score
    ctx.close()


def test_fused_attention_rejects_unsupported_shapes():
    from flutter_ml_b200 import _lib
    ctx = _lib.Context()
    buf, out = ctx.zeros(128, 3 * 64), ctx.zeros(128, 64)
    d = attention_desc(ctx, buf, out, None, 1, 128, 1, True, 0.125)
    d.d_head = 32
    assert ctx.lib.fml_attention_fwd(ctx.h, C.byref(d)) == -1
    d.d_head, d.seq_len = 64, 96
    assert ctx.lib.fml_attention_fwd(ctx.h, C.byref(d)) == -1
    ctx.close()


@pytest.mark.parametrize("S,causal", [(128, True), (256, True), (384, False), (512, True)])
@pytest.mark.parametrize("accumulate", [0, 1])
def test_fused_attention_backward(orc, S, causal, accumulate):
    """dQ, dK, dV of the fused backward against the oracle's tape for the same head: matMul, transpose,
    scale_matrix, softmax_matrix, matMul with an arbitrary upstream gradient."""
    from flutter_ml_b200 import _lib
    if accumulate and S != 256:
        pytest.skip("accumulation is shape-independent")
    ctx = _lib.Context(precision=_lib.PREC_TF32)
    Bn, H, dk = 2, 2, 64
    dm = H * dk
    rng = np.random.default_rng(7 * S + causal)
    qkv = rng.standard_normal((Bn * S, 3 * dm)).astype(np.float32)
    G = rng.standard_normal((Bn * S, dm)).astype(np.float32)
    scale = 1 / math.sqrt(dk)
    dq, out, lse, dG = ctx.upload(qkv), ctx.empty(Bn * S, dm), ctx.empty(Bn * H * S), ctx.upload(G)
    d = attention_desc(ctx, dq, out, lse, Bn, S, H, causal, scale)
    ctx.check(ctx.lib.fml_attention_fwd(ctx.h, C.byref(d)))
    base = rng.standard_normal((Bn * S, 3 * dm)).astype(np.float32) if accumulate else np.zeros((Bn * S, 3 * dm), np.float32)
    dqkv = ctx.upload(base)
    scratch = ctx.empty(Bn * H * S)
    ctx.check(ctx.lib.fml_attention_bwd(ctx.h, C.byref(d), dG.ptr, dm, dqkv.ptr, dqkv.ptr + 4 * dm, dqkv.ptr + 8 * dm, 3 * dm,
                                        accumulate, scratch.ptr))
    assert ctx.device_status() == 0
    got = dqkv.numpy() - base
    o_dev, lse_dev = out.numpy(), lse.numpy().reshape(Bn, H, S)
    E = orc.Engine(omp=True)
    for b in range(Bn):
        for h in range(H):
            rows = slice(b * S, (b + 1) * S)
            Q, K, V = (orc.T(w64(qkv[rows, i * dm + h * dk:i * dm + (h + 1) * dk])) for i in range(3))
            P = E.softmaxMatrix(E.scaleMatrix(E.matMul(Q, E.transpose(K)), scale), causal)
            O = E.matMul(P, V)
            E.sum(E.elementWiseMultiply(O, orc.T(w64(G[rows, h * dk:(h + 1) * dk])))).backward()
            cols = slice(h * dk, (h + 1) * dk)
            emu = emulate_backward(*(qkv[rows, i * dm + h * dk:i * dm + (h + 1) * dk] for i in range(3)), G[rows, cols],
                                   o_dev[rows, cols], lse_dev[b, h], scale, causal)
            for i, t in enumerate((Q, K, V)):
                g = got[rows, i * dm + h * dk:i * dm + (h + 1) * dk]
                # exact float64 chain (three truncating products deep for dQ and dK); with accumulate the difference of
                # two large numbers is compared, hence the wider bound
                assert rel(g, t.grad) <= (5e-3 if not accumulate else 2e-2), (b, h, "qkv"[i])
                if not accumulate:   # each backward product on the device's own inputs
                    assert rel(g, emu[i]) <= 3e-4, (b, h, "qkv"[i], rel(g, emu[i]))
    ctx.close()


def test_fused_attention_full_size_properties():
    """One config-5 layer (32 sequences x 16 heads x 512 x 64, causal), too large for the float64 oracle: properties
    that hold at any size.  With V = 1 every output equals 1 (the probabilities of a row sum to 1); the first query of
    a causal sequence sees only key 0, so its output row is V[0]; dV summed over keys equals dO summed over queries
    (each probability row sums to 1), and dQ, dK vanish when V is constant (dP is constant along a row, so dS = 0)."""
    from flutter_ml_b200 import _lib
    ctx = _lib.Context(precision=_lib.PREC_TF32)
    Bn, S, H, dk = 32, 512, 16, 64
    dm = H * dk
    rng = np.random.default_rng(99)
    qkv = rng.standard_normal((Bn * S, 3 * dm), dtype=np.float32)
    qkv[:, 2 * dm:] = 1.0
    G = rng.standard_normal((Bn * S, dm), dtype=np.float32)
    dq, out, lse, dG = ctx.upload(qkv), ctx.empty(Bn * S, dm), ctx.empty(Bn * H * S), ctx.upload(G)
    d = attention_desc(ctx, dq, out, lse, Bn, S, H, True, 0.125)
    ctx.check(ctx.lib.fml_attention_fwd(ctx.h, C.byref(d)))
    o = out.numpy()
    assert np.max(np.abs(o - 1.0)) <= 1e-5
    dqkv, scratch = ctx.empty(Bn * S, 3 * dm), ctx.empty(Bn * H * S)
    ctx.check(ctx.lib.fml_attention_bwd(ctx.h, C.byref(d), dG.ptr, dm, dqkv.ptr, dqkv.ptr + 4 * dm, dqkv.ptr + 8 * dm, 3 * dm, 0,
                                        scratch.ptr))
    g = dqkv.numpy()
    assert np.max(np.abs(g[:, :2 * dm])) <= 5e-3 * np.max(np.abs(G))          # dQ = dK = 0 up to the TF32 rounding of dO in dP
    dv_sum = g[:, 2 * dm:].reshape(Bn, S, dm).sum(1)
    do_sum = G.reshape(Bn, S, dm).astype(np.float64).sum(1)
    assert rel(dv_sum, do_sum) <= 1e-3
    # random V again: the first query of every sequence attends to key 0 only
    qkv[:, 2 * dm:] = rng.standard_normal((Bn * S, dm), dtype=np.float32)
    dq2 = ctx.upload(qkv)
    d2 = attention_desc(ctx, dq2, out, lse, Bn, S, H, True, 0.125)
    ctx.check(ctx.lib.fml_attention_fwd(ctx.h, C.byref(d2)))
    o = out.numpy().reshape(Bn, S, dm)
    v = qkv[:, 2 * dm:].reshape(Bn, S, dm)
    assert rel(o[:, 0, :], v[:, 0, :]) <= 1e-3        # one TF32 rounding of V
    # Every CTA works through about fourteen tiles here (one each in the small cases above), so where a tile lands is part of
    # what is tested: whole heads, spread over the batch, against exact float64 attention, forward and backward.
    ctx.check(ctx.lib.fml_attention_bwd(ctx.h, C.byref(d2), dG.ptr, dm, dqkv.ptr, dqkv.ptr + 4 * dm, dqkv.ptr + 8 * dm, 3 * dm, 0,
                                        scratch.ptr))
    g = dqkv.numpy()
    tril = np.tril(np.ones((S, S), bool))
    picks = [(0, 0), (Bn - 1, H - 1)] + [(int(rng.integers(Bn)), int(rng.integers(H))) for _ in range(8)]
    for b, h in picks:
        rows, cols = slice(b * S, (b + 1) * S), slice(h * dk, (h + 1) * dk)
        Q, K, V = (w64(qkv[rows, i * dm + h * dk:i * dm + (h + 1) * dk]) for i in range(3))
        sc = np.where(tril, Q @ K.T * 0.125, -np.inf)
        P = np.exp(sc - sc.max(1, keepdims=True))
        P /= P.sum(1, keepdims=True)
        dO = w64(G[rows, cols])
        dP = dO @ V.T
        dS = P * (dP - (dP * P).sum(1, keepdims=True)) * 0.125
        assert rel(o[b][:, cols], P @ V) <= 2e-3, (b, h)
        assert rel(g[rows, h * dk:(h + 1) * dk], dS @ K) <= 5e-3, (b, h)
        assert rel(g[rows, dm + h * dk:dm + (h + 1) * dk], dS.T @ Q) <= 5e-3, (b, h)
        assert rel(g[rows, 2 * dm + h * dk:2 * dm + (h + 1) * dk], P.T @ dO) <= 5e-3, (b, h)
    assert ctx.device_status() == 0
    ctx.close()
