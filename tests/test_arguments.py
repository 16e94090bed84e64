"""Argument validation and operator discovery (host logic; no GPU needed).  Mirrors the
reference's operators/test/unit/test_arguments.py and the rejection cases of
operators/test/integration/test_blockscaled_gemm.py."""
import pytest
import torch

import cutlass_b200 as ops
from cutlass_b200 import lib as L

SW = ops.ScaleSwizzleMode.Swizzle32x4x4
M16 = ops.ScaleMode.Blockwise1x16
M32 = ops.ScaleMode.Blockwise1x32


def nvfp4_args(M=256, N=256, K=512, L_=None, **kw):
    lead = () if L_ is None else (L_,)
    n = 1 if L_ is None else L_
    qa = torch.zeros(lead + (M, K // 2), dtype=torch.uint8)
    qb = torch.zeros(lead + (N, K // 2), dtype=torch.uint8).transpose(-1, -2)
    sa = torch.zeros(ops.ScaledOperand.numel_scale((n, M, K), M16, SW), dtype=torch.uint8)
    sb = torch.zeros(ops.ScaledOperand.numel_scale((n, N, K), M16, SW), dtype=torch.uint8)
    out = torch.zeros(lead + (M, N), dtype=torch.bfloat16)
    return ops.GemmArguments(ops.ScaledOperand(qa, sa, M16, SW), ops.ScaledOperand(qb, sb, M16, SW), out, torch.float32, **kw)


def mxfp8_args(M=128, N=384, K=256):
    qa = torch.zeros((M, K), dtype=torch.float8_e4m3fn)
    qb = torch.zeros((N, K), dtype=torch.float8_e4m3fn).t()
    sa = torch.zeros(ops.ScaledOperand.numel_scale((M, K), M32, SW), dtype=torch.uint8)
    sb = torch.zeros(ops.ScaledOperand.numel_scale((N, K), M32, SW), dtype=torch.uint8)
    return ops.GemmArguments(ops.ScaledOperand(qa, sa, M32, SW), ops.ScaledOperand(qb, sb, M32, SW),
                             torch.zeros((M, N), dtype=torch.bfloat16), torch.float32)


def test_numel_scale_formula():
    f = ops.ScaledOperand.numel_scale
    assert f((8192, 8192), M16, SW) == 8192 * 512
    assert f((2, 130, 100), M32, SW) == 2 * 256 * 4
    assert f((130, 100), M32, ops.ScaleSwizzleMode.SwizzleNone) == 130 * 4
    assert f((1, 1, 16), (1, 1, 16), SW) == 128 * 4
    with pytest.raises(ValueError):
        f((4,), M16, SW)
    assert ops.ScaleMode.compare(M16, (1, 1, 16)) and not ops.ScaleMode.compare(M16, M32)


def test_problem_size_accounts_for_fp4_packing():
    ps = nvfp4_args(M=256, N=384, K=512, L_=3).problem_size
    assert (ps.L, ps.M, ps.N, ps.K) == (3, 256, 384, 512)
    ps = mxfp8_args().problem_size
    assert (ps.L, ps.M, ps.N, ps.K) == (1, 128, 384, 256)


def test_shape_mismatches_raise():
    qa = torch.zeros((64, 64), dtype=torch.uint8)
    s = torch.zeros(128 * 8, dtype=torch.uint8)
    A = ops.ScaledOperand(qa, s, M16, SW)
    with pytest.raises(ValueError, match="contraction extents differ"):
        ops.GemmArguments(A, ops.ScaledOperand(torch.zeros((64, 32), dtype=torch.uint8).t(), s, M16, SW),
                          torch.zeros((64, 64), dtype=torch.bfloat16), torch.float32)
    B = ops.ScaledOperand(torch.zeros((64, 64), dtype=torch.uint8).t(), s, M16, SW)
    with pytest.raises(ValueError, match="out is 32 x 64 but A @ B is 64 x 64"):
        ops.GemmArguments(A, B, torch.zeros((32, 64), dtype=torch.bfloat16), torch.float32)
    with pytest.raises(ValueError, match="out is 64 x 48 but A @ B is 64 x 64"):
        ops.GemmArguments(A, B, torch.zeros((64, 48), dtype=torch.bfloat16), torch.float32)
    with pytest.raises(ValueError, match="rank"):
        ops.GemmArguments(A, B, torch.zeros((64,), dtype=torch.bfloat16), torch.float32)
    with pytest.raises(ValueError, match="batch"):
        ops.GemmArguments(ops.ScaledOperand(torch.zeros((2, 64, 64), dtype=torch.uint8), s, M16, SW), B,
                          torch.zeros((64, 64), dtype=torch.bfloat16), torch.float32)


def test_get_operators_orders_and_filters():
    found = ops.get_operators(nvfp4_args())
    assert [type(o) for o in found] == [ops.BlockScaledGemmOperator] * 6
    assert [(o.metadata.cta_group, o.metadata.tile_n) for o in found][4:] == [(2, 192), (2, 64)]
    assert (found[0].metadata.cta_group, found[0].metadata.tile_n) == (2, 256)
    assert all(o.metadata.kind == L.KIND_NVFP4 for o in found)
    only = ops.get_operators(nvfp4_args(), metadata_filter=lambda m: m.tile_n == 128 and m.cta_group == 1)
    assert len(only) == 1 and only[0].metadata.tile_shape == (128, 128, 256)
    assert all(o.metadata.kind == L.KIND_MXFP8 for o in ops.get_operators(mxfp8_args()))
    assert ops.get_operators(nvfp4_args(), target_sm="90a") == []
    # 2 kinds x 6 tile shapes + 2 kinds (MXFP4, MXFP8 x MXFP4) x 2 two-CTA tile shapes, each dense and grouped
    assert len(ops.all_operators()) == 32 and len({o.metadata.operator_name for o in ops.all_operators()}) == 32
    # the narrow tiles write bf16 or re-quantised outputs only
    f32 = nvfp4_args()
    f32.out = ops.DenseTensor(torch.zeros((256, 256), dtype=torch.float32))
    assert sorted((o.metadata.cta_group, o.metadata.tile_n) for o in ops.get_operators(f32)) == [(2, 128), (2, 256)]


def test_supports_rejections():
    op = ops.get_operators(nvfp4_args())[0]
    ok = nvfp4_args()
    assert op.supports(ok)
    # wrong swizzle
    bad = nvfp4_args()
    bad.A.swizzle = ops.ScaleSwizzleMode.SwizzleNone
    assert "swizzle" in str(op.supports(bad).error)
    # wrong scale numel
    bad = nvfp4_args()
    bad.A.scale = ops.DenseTensor(torch.zeros(17, dtype=torch.uint8))
    assert "scale tensor has 17 elements" in str(op.supports(bad).error)
    # mismatched modes between A and B
    bad = nvfp4_args()
    bad.B.mode = M32
    assert not op.supports(bad)
    # MN-major fp4 operand
    bad = nvfp4_args()
    bad.A.quantized = ops.DenseTensor(torch.zeros((256, 256), dtype=torch.uint8).t())
    assert "K-major" in str(op.supports(bad).error)
    # B given as a plain (K, N) contiguous tensor is not K-major
    bad = nvfp4_args()
    bad.B.quantized = ops.DenseTensor(torch.zeros((256, 256), dtype=torch.uint8))
    assert "K-major" in str(op.supports(bad).error)
    # accumulator type
    bad = nvfp4_args()
    bad.accumulator_type = torch.float16
    assert "accumulator" in str(op.supports(bad).error)
    # output dtype
    bad = nvfp4_args()
    bad.out = ops.DenseTensor(torch.zeros((256, 256), dtype=torch.float64))
    assert "out dtype" in str(op.supports(bad).error)
    # fp16 and fp32 outputs are taken as they are
    for dt in (torch.float16, torch.float32):
        good = nvfp4_args()
        good.out = ops.DenseTensor(torch.zeros((256, 256), dtype=dt))
        assert op.supports(good)
    # beta without C
    assert "beta" in str(op.supports(nvfp4_args(epilogue=ops.EpilogueDescriptor(beta=0.5))).error)
    # dense operands are not block-scaled
    dense = ops.GemmArguments(torch.zeros((64, 64), dtype=torch.bfloat16), torch.zeros((64, 64), dtype=torch.bfloat16),
                              torch.zeros((64, 64), dtype=torch.bfloat16), torch.float32)
    assert "ScaledOperand" in str(op.supports(dense).error)
    # operator of the other format
    assert not ops.all_operators()[-2].supports(ok)
    # run() raises ValueError for unsupported arguments before touching the library
    with pytest.raises(ValueError, match="does not support"):
        op.run(bad)


def test_nvfp4_output_descriptor_checks():
    M, N, K = 256, 256, 512
    sfd = torch.zeros(ops.ScaledOperand.numel_scale((M, N), M16, SW), dtype=torch.uint8)
    nc = torch.ones(1, dtype=torch.float32)
    a = nvfp4_args(M, N, K)
    args = ops.GemmArguments(a.A, a.B, torch.zeros((M, N // 2), dtype=torch.uint8), torch.float32,
                             epilogue=ops.EpilogueDescriptor(out_quant=ops.Nvfp4Quant(sfd, nc)))
    op = ops.get_operators(args)[0]
    assert op.supports(args)
    built = op.build_args(args)
    assert built.out_kind == L.OUT_NVFP4 and built.N == N and built.SFD == sfd.data_ptr()
    args.epilogue.out_quant.scale = torch.zeros(5, dtype=torch.uint8)
    assert "out_quant.scale" in str(op.supports(args).error)


def test_build_args_fills_the_abi_struct():
    c = torch.zeros((256, 256), dtype=torch.bfloat16)
    args = nvfp4_args(epilogue=ops.EpilogueDescriptor(alpha=2.0, beta=0.5, C=c))
    op = ops.get_operators(args, metadata_filter=lambda m: m.tile_n == 128 and m.cta_group == 2)[0]
    a = op.build_args(args)
    assert (a.kind, a.out_kind, a.batch, a.M, a.N, a.K) == (0, 0, 1, 256, 256, 512)
    assert a.A == args.A.quantized.data_ptr() and a.SFB == args.B.scale.data_ptr() and a.C == c.data_ptr()
    assert (a.alpha, a.beta, a.tile_n, a.cta_group, a.ldd) == (2.0, 0.5, 128, 2, 256)
    assert op.get_workspace_size(args).size_bytes == 16


def test_grouped_arguments_and_support():
    G_, N, K, total = 3, 256, 512, 700
    qa = torch.zeros((total, K // 2), dtype=torch.uint8)
    qb = torch.zeros((G_, N, K // 2), dtype=torch.uint8).transpose(-1, -2)
    sa = torch.zeros((5 + 3) * 128 * (K // 16), dtype=torch.uint8)      # between ceil(700/128) and 700//128 + groups atoms
    sb = torch.zeros(ops.ScaledOperand.numel_scale((G_, N, K), M16, SW), dtype=torch.uint8)
    out = torch.zeros((total, N), dtype=torch.bfloat16)
    offs = torch.tensor([100, 400, 700], dtype=torch.int32)
    args = ops.GroupedGemmArguments(ops.ScaledOperand(qa, sa, M16, SW), ops.ScaledOperand(qb, sb, M16, SW), out, torch.float32, offs)
    found = ops.get_operators(args)
    assert found and all(isinstance(o, ops.GroupedBlockScaledGemmOperator) for o in found)
    a = found[0].build_args(args)
    assert (a.num_groups, a.total_M, a.N, a.K, a.offsets) == (3, 700, 256, 512, offs.data_ptr())
    with pytest.raises(ValueError, match="int32"):
        ops.GroupedGemmArguments(args.A, args.B, out, torch.float32, offs.to(torch.int64))
    with pytest.raises(ValueError, match="entries"):
        ops.GroupedGemmArguments(args.A, args.B, out, torch.float32, offs[:2])
    with pytest.raises(ValueError, match="offsets is required"):
        ops.GroupedGemmArguments(args.A, args.B, out, torch.float32)
    args.A.scale = ops.DenseTensor(torch.zeros(128, dtype=torch.uint8))
    assert "scale tensor" in str(found[0].supports(args).error)


def test_status_object():
    assert ops.Status.success() and not ops.Status.fail("x")
    with pytest.raises(ValueError, match="boom"):
        ops.Status.fail("boom").raise_on_error()


def test_stream_conversion():
    assert ops.to_cuda_stream(None) == 0 and ops.to_cuda_stream(17) == 17

    class S:
        cuda_stream = 99
    assert ops.to_cuda_stream(S()) == 99
    with pytest.raises(TypeError):
        ops.to_cuda_stream(object())


def test_mxfp8_output_descriptor_checks():
    M, N, K = 256, 256, 512
    sfd = torch.zeros(ops.ScaledOperand.numel_scale((M, N), M32, SW), dtype=torch.uint8)
    a = nvfp4_args(M, N, K)
    args = ops.GemmArguments(a.A, a.B, torch.zeros((M, N), dtype=torch.uint8), torch.float32,
                             epilogue=ops.EpilogueDescriptor(out_quant=ops.Mxfp8Quant(sfd)))
    assert not args.out_is_packed_fp4
    op = ops.get_operators(args)[0]
    assert op.supports(args)
    built = op.build_args(args)
    assert built.out_kind == L.OUT_MXFP8 and built.N == N and built.SFD == sfd.data_ptr() and not built.norm_constant
    args.epilogue.out_quant.scale = torch.zeros(7, dtype=torch.uint8)
    assert "out_quant.scale" in str(op.supports(args).error)
    args.epilogue.out_quant = ops.Mxfp8Quant(sfd, norm_constant=torch.ones(2, dtype=torch.float32))
    assert "norm_constant" in str(op.supports(args).error)


def test_bias_and_activation_descriptor():
    M, N, K = 256, 384, 512
    bias_n, bias_m = torch.zeros(N, dtype=torch.float32), torch.zeros(M, dtype=torch.float32)
    args = nvfp4_args(M, N, K, epilogue=ops.EpilogueDescriptor(bias=bias_n, activation="gelu"))
    op = ops.get_operators(args)[0]
    assert op.supports(args)
    a = op.build_args(args)
    assert (a.bias, a.bias_mode, a.activation) == (bias_n.data_ptr(), L.BIAS_PER_COLUMN, L.ACT_GELU)
    args = nvfp4_args(M, N, K, epilogue=ops.EpilogueDescriptor(bias=bias_m, bias_per_row=True, activation="silu"))
    a = op.build_args(args)
    assert op.supports(args) and (a.bias_mode, a.activation) == (L.BIAS_PER_ROW, L.ACT_SILU)
    assert op.build_args(nvfp4_args(M, N, K)).bias_mode == L.BIAS_NONE
    bad = nvfp4_args(M, N, K, epilogue=ops.EpilogueDescriptor(bias=bias_m))            # M entries for a per-column bias
    assert "bias" in str(op.supports(bad).error)
    bad = nvfp4_args(M, N, K, epilogue=ops.EpilogueDescriptor(bias=bias_n.double()))
    assert "bias" in str(op.supports(bad).error)
    bad = nvfp4_args(M, N, K, epilogue=ops.EpilogueDescriptor(activation="tanh"))
    assert "activation" in str(op.supports(bad).error)


def test_abi_rejects_bad_bias_and_activation():
    lib = L.load()
    a = L.GemmArgs()
    a.kind, a.batch, a.M, a.N, a.K = 0, 1, 256, 256, 256
    a.A = a.B = a.SFA = a.SFB = a.D = 0x10000
    a.alpha = 1.0
    caps = L.Caps()
    a.activation = 9
    assert lib.bsg_gemm_query(a, caps) == 3                     # BSG_ERR_NOT_SUPPORTED
    a.activation, a.bias_mode = 1, 1
    assert lib.bsg_gemm_query(a, caps) == 2                     # bias mode without a bias vector
    a.bias = 0x10004
    assert lib.bsg_gemm_query(a, caps) == 1                     # misaligned bias
    a.bias = 0x10000
    assert lib.bsg_gemm_query(a, caps) == 0


def test_quantize_blockscaled_argument_checks():
    x = torch.zeros((64, 128), dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="CUDA"):
        ops.quantize_blockscaled(x, M16)
    with pytest.raises(ValueError, match="scale mode"):
        ops.quantize_blockscaled(x, (1, 1, 64))


def test_get_operators_takes_the_reference_parameters():
    args = nvfp4_args()
    everything = ops.get_operators(args)
    assert len(ops.get_operators(args, None, "100a", [ops.NativeProvider])) == len(everything)
    assert len(ops.get_operators(args, providers=[ops.NativeProvider])) == len(everything) > 0
    assert ops.get_operators(args, providers=[]) == []
    assert ops.get_operators(args, target_sm="90a") == []


def test_mxfp4_and_mixed_pairs_are_discovered():
    """MXFP4 needs the packed fp4 dtype (uint8 with 32-wide blocks means e4m3 codes); MXFP8 A with MXFP4 B is the mixed kind."""
    fp4 = getattr(torch, "float4_e2m1fn_x2", None)
    if fp4 is None:
        pytest.skip("this torch has no packed fp4 dtype")
    M, N, K = 128, 256, 256
    sa = torch.zeros(ops.ScaledOperand.numel_scale((M, K), M32, SW), dtype=torch.uint8)
    sb = torch.zeros(ops.ScaledOperand.numel_scale((N, K), M32, SW), dtype=torch.uint8)
    a4 = ops.ScaledOperand(torch.zeros((M, K // 2), dtype=torch.uint8).view(fp4), sa, M32, SW)
    a8 = ops.ScaledOperand(torch.zeros((M, K), dtype=torch.uint8), sa, M32, SW)
    b4 = ops.ScaledOperand(torch.zeros((N, K // 2), dtype=torch.uint8).view(fp4).t(), sb, M32, SW)
    out = torch.zeros((M, N), dtype=torch.bfloat16)
    found = ops.get_operators(ops.GemmArguments(a4, b4, out, torch.float32))
    assert found and all(o.metadata.kind == L.KIND_MXFP4 and o.metadata.cta_group == 2 for o in found)
    found = ops.get_operators(ops.GemmArguments(a8, b4, out, torch.float32))
    assert found and all(o.metadata.kind == L.KIND_MXFP8_MXFP4 for o in found)
    # the other way round (MXFP4 A with MXFP8 B) has no kernel
    b8 = ops.ScaledOperand(torch.zeros((N, K), dtype=torch.uint8).t(), sb, M32, SW)
    assert ops.get_operators(ops.GemmArguments(a4, b8, out, torch.float32)) == []


def test_row_pitch_and_batch_stride_reach_the_abi():
    """A slice of a larger buffer (row pitch > K, batch entries further apart than one matrix) is accepted and its
    strides arrive in bsg_gemm_args in logical elements."""
    Lb, M, N, K = 2, 128, 128, 256
    big = torch.zeros((Lb, M + 8, K // 2 + 32), dtype=torch.uint8)
    A = ops.ScaledOperand(big[:, :M, :K // 2], torch.zeros(ops.ScaledOperand.numel_scale((Lb, M, K), M16, SW), dtype=torch.uint8), M16, SW)
    B = ops.ScaledOperand(torch.zeros((Lb, N, K // 2), dtype=torch.uint8).transpose(1, 2),
                          torch.zeros(ops.ScaledOperand.numel_scale((Lb, N, K), M16, SW), dtype=torch.uint8), M16, SW)
    outbuf = torch.zeros((Lb, M, N + 16), dtype=torch.bfloat16)
    args = ops.GemmArguments(A, B, outbuf[:, :, :N], torch.float32)
    op = ops.get_operators(args)[0]
    abi = op.build_args(args)
    assert (abi.lda, abi.batch_stride_A) == ((K // 2 + 32) * 2, (M + 8) * (K // 2 + 32) * 2)
    assert (abi.ldb, abi.batch_stride_B) == (K, N * K)
    assert (abi.ldd, abi.batch_stride_D) == (N + 16, M * (N + 16))
    # a row pitch that breaks the 16-byte alignment is refused
    odd = torch.zeros((M, K // 2 + 8), dtype=torch.uint8)[:, :K // 2]
    bad = ops.GemmArguments(ops.ScaledOperand(odd, torch.zeros(ops.ScaledOperand.numel_scale((M, K), M16, SW), dtype=torch.uint8), M16, SW),
                            ops.ScaledOperand(torch.zeros((N, K // 2), dtype=torch.uint8).t(),
                                              torch.zeros(ops.ScaledOperand.numel_scale((N, K), M16, SW), dtype=torch.uint8), M16, SW),
                            torch.zeros((M, N), dtype=torch.bfloat16), torch.float32)
    assert ops.get_operators(bad) == []


def test_pointer_array_groups_are_checked_on_the_host():
    """GroupProblem tensors: K must agree between A and B, tensors are two-dimensional with a contiguous last dimension."""
    import torch
    from cutlass_b200 import lib as L
    from cutlass_b200.ptr_array import GroupProblem, PtrArrayGemm
    u8 = lambda *s: torch.zeros(s, dtype=torch.uint8)  # noqa: E731
    with pytest.raises(ValueError, match="disagree on K"):
        PtrArrayGemm(L.KIND_NVFP4, [GroupProblem(A=u8(128, 64), SFA=u8(512), B=u8(128, 32), SFB=u8(512), D=torch.zeros((128, 128), dtype=torch.bfloat16))])
    with pytest.raises(ValueError, match="contiguous last dimension"):
        PtrArrayGemm(L.KIND_MXFP8, [GroupProblem(A=u8(128, 256)[:, ::2], SFA=u8(512), B=u8(128, 128), SFB=u8(512),
                                                 D=torch.zeros((128, 128), dtype=torch.bfloat16))])
    with pytest.raises(ValueError, match="at least one group"):
        PtrArrayGemm(L.KIND_MXFP8, [])
