"""vx_bsgemm_residual_ln: the residual GEMM with the next LayerNorm + MX32 quantizer in its epilogue (a cluster
of two CTAs per 128 rows) against the two separate launches it replaces, bit for bit, and against the CPU oracle."""

import numpy as np
import pytest
import torch

from oracle import formats as F
from oracle import gemm as G

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from velox_voice_b200 import ops as o

    return o


def _case(M, K, seed, scale=1.0):
    from velox_voice_b200.linear import PackedLinear

    g = torch.Generator().manual_seed(seed)
    a = (torch.randn(M, K, generator=g) * scale).bfloat16().cuda()
    w = torch.randn(512, K, generator=g) * 0.05
    bias = torch.randn(512, generator=g) * 0.1
    res = torch.randn(M, 512, generator=g).bfloat16().cuda()
    gamma = (1.0 + 0.2 * torch.randn(512, generator=g)).cuda()
    beta = (0.1 * torch.randn(512, generator=g)).cuda()
    lin = PackedLinear(w.cuda(), bias.cuda(), "mx32")
    return a, lin, res, gamma, beta


@pytest.mark.parametrize("M,K,alpha", [(1, 512, 1.0), (100, 512, 0.5), (128, 256, 1.0), (129, 512, 1.0), (300, 2048, 0.5),
                                        (1000, 512, 1.0), (9473, 512, 1.0), (9473, 2048, 0.5), (20000, 768, 1.0)])
def test_fused_equals_gemm_then_ln_quantize(ops, M, K, alpha):
    """x, codes and scale-factor atoms equal those of bsgemm(BIAS_RESIDUAL) followed by ln_quantize: bit-exact."""
    a, lin, res, gamma, beta = _case(M, K, seed=M + K)
    qa = ops.quantize(a, "mx32")
    assert lin.residual_ln_supported()
    x_ref = lin(qa, residual=res, alpha=alpha)
    q_ref = ops.ln_quantize(x_ref, gamma, beta, 1e-5, "mx32")
    x, q = lin.residual_ln(qa, residual=res, gamma=gamma, beta=beta, eps=1e-5, alpha=alpha)
    torch.cuda.synchronize()
    assert x.dtype == torch.bfloat16 and x.shape == (M, 512)
    assert torch.equal(x, x_ref)
    assert torch.equal(q.codes, q_ref.codes)
    assert torch.equal(q.sf, q_ref.sf)


@pytest.mark.parametrize("M,K,alpha", [(1, 512, 1.0), (129, 2048, 0.5), (1000, 2048, 0.5), (9473, 2048, 0.5), (20000, 512, 1.0)])
def test_fused_two_layernorms_equal_gemm_then_ln2_quantize(ops, M, K, alpha):
    """The end of a block: y = LN(x) stored over the residual stream and quantize(LN(y)) equal, bit for bit,
    bsgemm(BIAS_RESIDUAL) followed by ln2_quantize(y=x)."""
    a, lin, res, gamma, beta = _case(M, K, seed=M + K + 1)
    g = torch.Generator().manual_seed(M)
    gamma2 = (1.0 + 0.2 * torch.randn(512, generator=g)).cuda()
    beta2 = (0.1 * torch.randn(512, generator=g)).cuda()
    qa = ops.quantize(a, "mx32")
    x_ref = lin(qa, residual=res, alpha=alpha)
    q_ref = ops.ln2_quantize(x_ref, gamma, beta, gamma2, beta2, 1e-5, "mx32", y=x_ref)  # x_ref now holds y
    buf = res.clone()
    y, q = lin.residual_ln(qa, residual=buf, gamma=gamma, beta=beta, eps=1e-5, alpha=alpha, out=buf, gamma2=gamma2, beta2=beta2)
    torch.cuda.synchronize()
    assert y.data_ptr() == buf.data_ptr()
    assert torch.equal(y, x_ref)
    assert torch.equal(q.codes, q_ref.codes)
    assert torch.equal(q.sf, q_ref.sf)


def test_fused_in_place_and_repeated(ops):
    """out aliases the residual (the encoder's residual stream), two layers in a row."""
    M = 3000
    a, lin, res, gamma, beta = _case(M, 512, seed=5)
    qa = ops.quantize(a, "mx32")
    x_ref = lin(qa, residual=res.clone(), alpha=1.0)
    q_ref = ops.ln_quantize(x_ref, gamma, beta, 1e-5, "mx32")
    x2_ref = lin(q_ref, residual=x_ref.clone(), alpha=0.5)
    q2_ref = ops.ln_quantize(x2_ref, gamma, beta, 1e-5, "mx32")
    x = res.clone()
    x1, q1 = lin.residual_ln(qa, residual=x, gamma=gamma, beta=beta, eps=1e-5, alpha=1.0, out=x)
    assert x1.data_ptr() == x.data_ptr()
    x2, q2 = lin.residual_ln(q1, residual=x, gamma=gamma, beta=beta, eps=1e-5, alpha=0.5, out=x)
    torch.cuda.synchronize()
    assert torch.equal(x2, x2_ref)
    assert torch.equal(q2.codes, q2_ref.codes) and torch.equal(q2.sf, q2_ref.sf)


def test_fused_matches_the_oracle(ops):
    """x within the path's bound of the oracle GEMM + epilogue; codes and scales bit-exact against the oracle's
    LayerNorm (half-row summation order) + MX32 quantizer applied to the x the kernel stored."""
    M, K = 200, 512
    a, lin, res, gamma, beta = _case(M, K, seed=11)
    qa = ops.quantize(a, "mx32")
    x, q = lin.residual_ln(qa, residual=res, gamma=gamma, beta=beta, eps=1e-5, alpha=0.5)
    torch.cuda.synchronize()
    wq = lin.q
    acc = G.gemm_ref(F.FMT_MX32, qa.codes.cpu().numpy(), qa.scales.cpu().numpy(), wq.codes.cpu().numpy(),
                     wq.scales.cpu().numpy())
    y = G.epilogue_ref(acc, G.EPI_BIAS_RESIDUAL, lin.bias.cpu().numpy(), res.float().cpu().numpy(), 0.5)
    xg = x.float().cpu().numpy()
    assert float(np.abs(xg - y).max() / np.abs(y).max()) < 1e-2
    ln = G.layernorm_ref(xg, gamma.cpu().numpy(), beta.cpu().numpy(), 1e-5, half_rows=True)
    oc, osc, _ = F.quantize(ln, F.FMT_MX32)
    assert np.array_equal(q.codes.cpu().numpy(), oc)
    assert np.array_equal(q.sf.cpu().numpy(), F.sf_atoms(osc))


def test_argument_checks(ops):
    a, lin, res, gamma, beta = _case(64, 512, seed=3)
    qa = ops.quantize(a, "mx32")
    with pytest.raises(ValueError):
        lin.residual_ln(qa, residual=res[:, :256], gamma=gamma, beta=beta, eps=1e-5)
    assert not ops.residual_ln_supported("nv16", 512, 512)
    assert not ops.residual_ln_supported("mx32", 256, 512)
    assert not ops.residual_ln_supported("mx32", 512, 384)
    assert ops.residual_ln_supported("mx32", 512, 2048)


def test_stack_with_fused_layernorms_reproduces_the_oracle():
    """The 12-block MX32 stack with every eligible residual GEMM running the LayerNorm + quantizer behind it (no
    frame threshold): the same logits, bit for bit, as the stack with separate launches, and the CPU oracle's."""
    from velox_voice_b200 import _lib
    from velox_voice_b200.stack import ConformerLinearStack, StackConfig, make_weights
    from oracle.stack import OracleStack

    T = 1000
    cfg_f = StackConfig(blocks=12, fmt="mx32", fuse_ln=True, fuse_ln_min_frames=0)
    cfg_u = StackConfig(blocks=12, fmt="mx32", fuse_ln=False)
    w = make_weights(cfg_f, seed=0)
    # non-trivial LayerNorm parameters (make_weights leaves them at identity)
    g = torch.Generator().manual_seed(3)
    for k in list(w):
        if k.endswith(".g"):
            w[k] = 1.0 + 0.1 * torch.randn(w[k].shape, generator=g)
        elif k.endswith(".b") and ("ln_" in k or k.startswith("after")):
            w[k] = 0.05 * torch.randn(w[k].shape, generator=g)
    fused, plain = ConformerLinearStack(cfg_f, w), ConformerLinearStack(cfg_u, w)
    assert fused.fuse_ln and not plain.fuse_ln
    torch.manual_seed(0)
    x = torch.randn(T, cfg_f.d_model).bfloat16()
    pos = torch.randn(T, cfg_f.d_model).bfloat16().cuda()
    n0 = ops_count()
    lf = fused.forward(x.cuda().clone(), pos)
    n1 = ops_count()
    lu = plain.forward(x.cuda().clone(), pos)
    n2 = ops_count()
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert (n2 - n1) - (n1 - n0) == 4 * cfg_f.blocks  # four launches fewer per block
    assert torch.equal(lf, lu)
    ref = OracleStack({k: v.numpy() for k, v in w.items()}, F.FMT_NAMES["mx32"], cfg_f.blocks, fuse_ffn=fused.fuse_ffn).forward(x.float().numpy())
    got = lf.float().cpu().numpy()
    assert np.abs(got - ref).max() / np.abs(ref).max() < 1e-2
    assert float((got.argmax(1) == ref.argmax(1)).mean()) >= 0.999


def ops_count():
    from velox_voice_b200 import ops

    return ops.launch_count()
