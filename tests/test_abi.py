"""The C-ABI shared library: builds, loads without a GPU, exports every declared symbol,
and answers the calls that need no device."""
import ctypes as C
import os
import re

import pytest

from cutlass_b200 import build as B
from cutlass_b200 import lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    B.build()
    return L.load()


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "bsgemm.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bsg_[a-z_0-9]+)\s*\(", text)))


def test_header_symbols_are_all_exported(lib):
    names = _declared_symbols()
    assert len(names) >= 9
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/bsgemm.h but not exported"
    assert sorted(L.SYMBOLS) == names, "cutlass_b200.lib.SYMBOLS must list exactly the header's entry points"


def test_version_and_error_string(lib):
    assert lib.bsg_version() >= 100
    assert isinstance(lib.bsg_last_error_string(), bytes)


def test_struct_sizes_match_header_layout():
    # 4 int32, 3 int64, 7 pointers, 2 int64, 2 float, 3 pointers, 4 int32; bias pointer, bias_mode, activation;
    # lda, ldb and four batch strides (int64); use_pdl, scheduler and four cluster extents (int32)
    assert C.sizeof(L.GemmArgs) == 16 + 24 + 56 + 16 + 8 + 24 + 16 + 16 + 48 + 24 + 8      # + out_layout, reserved1
    # ... alpha_array, beta_array; SFD, norm_constant, use_pdl, scheduler
    assert C.sizeof(L.GroupedArgs) == 16 + 24 + 56 + 16 + 8 + 16 + 16 + 16 + 24
    assert C.sizeof(L.Caps) == 32
    # 4 int32, the sizes pointer, 7 pointer arrays, 4 pitch arrays, 2 floats, 3 pointers, 4 int32
    assert C.sizeof(L.PtrArrayArgs) == 16 + 8 + 56 + 32 + 8 + 24 + 16


def _args(**kw):
    a = L.GemmArgs()
    a.kind, a.out_kind, a.batch = 0, 0, 1
    a.M, a.N, a.K = 256, 256, 256
    for f in ("A", "B", "SFA", "SFB", "D"):
        setattr(a, f, 0x10000)      # never dereferenced by the query
    a.alpha = 1.0
    for k, v in kw.items():
        setattr(a, k, v)
    return a


def test_query_accepts_valid_problem_and_reports_plan(lib):
    caps = L.Caps()
    assert lib.bsg_gemm_query(C.byref(_args()), C.byref(caps)) == 0
    assert (caps.tile_m, caps.tile_n, caps.tile_k, caps.cta_group) == (256, 256, 256, 2)
    assert caps.stages >= 4 and caps.smem_bytes <= 232448 and caps.num_tiles == 1
    assert lib.bsg_gemm_query(C.byref(_args(kind=1, tile_n=128, cta_group=1)), C.byref(caps)) == 0
    assert (caps.tile_m, caps.tile_n, caps.tile_k) == (128, 128, 128) and caps.num_tiles == 4
    assert lib.bsg_gemm_query(C.byref(_args(N=384, tile_n=192)), C.byref(caps)) == 0
    assert (caps.tile_n, caps.num_tiles, caps.stages) == (192, 2, 5)
    assert lib.bsg_gemm_query(C.byref(_args(tile_n=64)), C.byref(caps)) == 0 and (caps.tile_n, caps.num_tiles) == (64, 4)


@pytest.mark.parametrize("kw,code", [
    (dict(K=48), 1),                 # K not a multiple of 32 for NVFP4
    (dict(kind=1, K=40), 1),         # K not a multiple of 16 for MXFP8
    (dict(A=0x10001), 1),            # misaligned pointer
    (dict(N=100), 1),                # bf16 rows not 16-byte multiples
    (dict(kind=7), 3),
    (dict(use_pdl=2), 2),
    (dict(tile_n=96), 3),
    (dict(tile_n=192, cta_group=1), 3),      # tiles of 64 / 192 columns need the 2-CTA form
    (dict(tile_n=64, scheduler=1), 3),
    (dict(cta_group=3), 3),
    (dict(N=0), 2),
    (dict(A=None), 2),
    (dict(beta=0.5), 2),             # beta without C
    (dict(out_kind=1), 2),           # NVFP4 output without SFD / norm constant
    (dict(batch=1000), 2),
    (dict(lda=128), 2),              # row pitch smaller than K
    (dict(lda=272), 1),              # row pitch that breaks the 16-byte row alignment (e2m1: multiples of 32)
    (dict(batch=2, batch_stride_A=256 * 256 + 8), 1),
    (dict(scheduler=5), 3),
    (dict(use_pdl=2), 2),
    (dict(cluster_m=2, cluster_n=4), 3),     # the reference's multicast cluster: nothing here uses it
])
def test_query_rejects_bad_problems(lib, kw, code):
    assert lib.bsg_gemm_query(C.byref(_args(**kw)), None) == code
    assert len(L.last_error()) > 0


def test_workspace_size_and_null_workspace(lib):
    n = C.c_size_t(0)
    assert lib.bsg_gemm_workspace_size(C.byref(_args()), C.byref(n)) == 0 and n.value == 16
    # run() validates before touching the device: a null workspace is reported, not dereferenced
    assert lib.bsg_gemm_run(C.byref(_args()), None, 0, None) == 4


def test_grouped_query(lib):
    g = L.GroupedArgs()
    g.kind, g.num_groups, g.total_M, g.N, g.K = 0, 4, 1000, 256, 512
    for f in ("A", "B", "SFA", "SFB", "D", "offsets"):
        setattr(g, f, 0x10000)
    g.alpha = 1.0
    caps = L.Caps()
    assert lib.bsg_grouped_query(C.byref(g), C.byref(caps)) == 0 and caps.num_tiles == -1
    g.num_groups = 1000
    assert lib.bsg_grouped_query(C.byref(g), None) == 2
    g.num_groups = 4
    g.offsets = None
    assert lib.bsg_grouped_query(C.byref(g), None) == 2


def _quant_args(**kw):
    a = L.QuantArgs()
    a.kind, a.rows, a.K, a.ldx = 0, 256, 256, 256
    a.X = a.Q = a.SF = 0x10000          # rejected before anything is dereferenced or launched
    for k, v in kw.items():
        setattr(a, k, v)
    return a


@pytest.mark.parametrize("kw,code", [
    (dict(kind=7), 3),
    (dict(K=48, ldx=48), 1),        # K must be a multiple of 32
    (dict(ldx=250), 1),             # shorter than K
    (dict(ldx=260), 1),             # rows not 16-byte aligned
    (dict(rows=-1), 2),
    (dict(X=None), 2),
    (dict(SF=0x10004), 1),
])
def test_quantiser_rejects_bad_arguments_before_launching(lib, kw, code):
    assert C.sizeof(L.QuantArgs) == 8 + 16 + 8 + 8 + 24
    assert lib.bsg_quantize(C.byref(_quant_args(**kw)), None) == code
    assert lib.bsg_last_error_string()


def test_quantiser_accepts_an_empty_matrix(lib):
    assert lib.bsg_quantize(C.byref(_quant_args(rows=0)), None) == L.BSG_OK


def _ptr_array_args(sizes, ptr=0x10000, **kw):
    n = len(sizes)
    keep = {"sizes": (C.c_int32 * (3 * n))(*[v for s in sizes for v in s])}
    a = L.PtrArrayArgs()
    a.kind, a.out_kind, a.num_groups = 0, 0, n
    a.problem_sizes = C.cast(keep["sizes"], C.c_void_p)
    for f in ("A", "B", "SFA", "SFB", "D"):
        keep[f] = (C.c_void_p * n)(*([ptr] * n))        # never dereferenced by the checks
        setattr(a, f, C.cast(keep[f], C.c_void_p))
    a.alpha = 1.0
    for k, v in kw.items():
        setattr(a, k, v)
    return a, keep


def test_pointer_array_form_checks_every_group_before_touching_the_device(lib):
    a, keep = _ptr_array_args([(300, 640, 512), (0, 256, 256), (64, 128, 256)])
    n = C.c_size_t(0)
    assert lib.bsg_ptr_array_workspace_size(C.byref(a), C.byref(n)) == 0 and n.value == 8192 + 3 * 768
    # all groups pass the checks: the next thing looked at is the workspace
    assert lib.bsg_ptr_array_initialize(C.byref(a), None, 0, None) == 4
    assert lib.bsg_ptr_array_initialize(C.byref(a), 0x10040, n.value, None) == 1 and "128-byte" in L.last_error()
    # a group whose K breaks the 16-byte row rule is named
    b, keep_b = _ptr_array_args([(300, 640, 512), (64, 128, 48)])
    assert lib.bsg_ptr_array_initialize(C.byref(b), None, 0, None) == 1 and L.last_error().startswith("group 1:")
    # a misaligned pointer in one group
    keep["B"][2] = 0x10008
    assert lib.bsg_ptr_array_initialize(C.byref(a), None, 0, None) == 1 and L.last_error().startswith("group 2:")
    keep["B"][2] = 0x10000
    # beta without C, unknown kinds, too many groups
    c, _k = _ptr_array_args([(128, 128, 128)], beta=1.0)
    assert lib.bsg_ptr_array_initialize(C.byref(c), None, 0, None) == 2
    d, _k2 = _ptr_array_args([(128, 128, 128)], kind=2)
    assert lib.bsg_ptr_array_initialize(C.byref(d), None, 0, None) == 3
    a.num_groups = 1000
    assert lib.bsg_ptr_array_workspace_size(C.byref(a), C.byref(n)) == 2
    a.num_groups = 3
    # a run needs a table: this workspace has never been initialised
    assert lib.bsg_ptr_array_run(C.byref(a), 0x20000, 1 << 20, None) == 2 and "initialize" in L.last_error()
