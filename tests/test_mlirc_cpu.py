"""The MLIR C API surface (include/mlir_c_b200.h) without a GPU: the builder calls and the pipeline / getter
sequence of the reference's C-API example (mlir/test/CAPI/mixr_full.c) in tests/mlirc_client.c, and the text front end
with the three pipelines on module texts written in the assembly the migraphx dialect prints
(mlir/include/mlir/Dialect/MIGraphX/IR/MIGraphX.td:38-588)."""
import glob
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

DOT_ADD = """
module {
  func.func @dot_add(%arg0: !migraphx.shaped<1x5x4xf32, 20x4x1>, %arg1: !migraphx.shaped<1x4x3xf32, 12x3x1>,
                     %arg2: !migraphx.shaped<1x5x3xf32, 15x3x1>) -> !migraphx.shaped<1x5x3xf32, 15x3x1> attributes{kernel, arch = "sm_100a"} {
    %0 = migraphx.dot %arg0, %arg1 : <1x5x4xf32, 20x4x1>, <1x4x3xf32, 12x3x1> -> <1x5x3xf32, 15x3x1>
    %2 = migraphx.add %0, %arg2 {} : <1x5x3xf32, 15x3x1>, <1x5x3xf32, 15x3x1> -> <1x5x3xf32, 15x3x1>
    return %2 : !migraphx.shaped<1x5x3xf32, 15x3x1>
  }
}
"""

# a transposed B (column-major strides) and a per-column bias through multibroadcast, f16
DOT_TRANSB_BIAS_RELU = """
func.func @mlir_dot_add_relu(%a: !migraphx.shaped<2x384x256xf16, 98304x256x1>, %b: !migraphx.shaped<2x256x520xf16, 133120x1x256>,
                             %bias: !migraphx.shaped<520xf16, 1>) -> !migraphx.shaped<2x384x520xf16, 199680x520x1> attributes {kernel = "mixr", arch = "sm_100a"} {
  %0 = migraphx.dot %a, %b : <2x384x256xf16, 98304x256x1>, <2x256x520xf16, 133120x1x256> -> <2x384x520xf16, 199680x520x1>
  %1 = migraphx.multibroadcast %bias {out_dyn_dims = [], out_lens = [2, 384, 520]} : <520xf16, 1> -> <2x384x520xf16, 0x0x1>
  %2 = migraphx.add %0, %1 : <2x384x520xf16, 199680x520x1>, <2x384x520xf16, 0x0x1> -> <2x384x520xf16, 199680x520x1>
  %3 = migraphx.relu %2 : <2x384x520xf16, 199680x520x1> -> <2x384x520xf16, 199680x520x1>
  return %3 : !migraphx.shaped<2x384x520xf16, 199680x520x1>
}
"""

# NHWC tensors expressed through strides; bias, clip with literal bounds
CONV_BIAS_CLIP_NHWC = """
module {
  func.func @mlir_convolution_add_clip(%bias: !migraphx.shaped<1x96x1x1xf16, 96x1x1x1>, %x: !migraphx.shaped<2x64x14x14xf16, 12544x1x896x64>,
                                       %w: !migraphx.shaped<96x64x3x3xf16, 576x1x192x64>) -> !migraphx.shaped<2x96x14x14xf16, 18816x1x1344x96> attributes {kernel, arch = "sm_100a"} {
    %0 = migraphx.multibroadcast %bias {out_dyn_dims = [], out_lens = [2, 96, 14, 14]} : <1x96x1x1xf16, 96x1x1x1> -> <2x96x14x14xf16, 0x1x0x0>
    %hi = migraphx.literal (dense<6.000000e+00> : tensor<1xf16>) : <1xf16, 0>
    %lo = migraphx.literal (dense<0.000000e+00> : tensor<1xf16>) : <1xf16, 0>
    %3 = migraphx.multibroadcast %lo {out_dyn_dims = [], out_lens = [2, 96, 14, 14]} : <1xf16, 0> -> <2x96x14x14xf16, 0x0x0x0>
    %4 = migraphx.multibroadcast %hi {out_dyn_dims = [], out_lens = [2, 96, 14, 14]} : <1xf16, 0> -> <2x96x14x14xf16, 0x0x0x0>
    %5 = migraphx.convolution %x, %w {dilation = [1, 1], group = 1 : i64, padding = [1, 1, 1, 1], padding_mode = 0 : i64, stride = [1, 1]} : <2x64x14x14xf16, 12544x1x896x64>, <96x64x3x3xf16, 576x1x192x64> -> <2x96x14x14xf16, 18816x1x1344x96>
    %6 = migraphx.add %5, %0 : <2x96x14x14xf16, 18816x1x1344x96>, <2x96x14x14xf16, 0x1x0x0> -> <2x96x14x14xf16, 18816x1x1344x96>
    %7 = migraphx.clip %6, %3, %4 : <2x96x14x14xf16, 18816x1x1344x96>, <2x96x14x14xf16, 0x0x0x0>, <2x96x14x14xf16, 0x0x0x0> -> <2x96x14x14xf16, 18816x1x1344x96>
    return %7 : !migraphx.shaped<2x96x14x14xf16, 18816x1x1344x96>
  }
}
"""

# quant_convolution -> dequantizelinear -> add (implicit broadcast of a 1xCx1x1 argument) -> relu -> quantizelinear
QUANT_CONV = """
module {
  func.func @mlir_quantization(%arg0: !migraphx.shaped<1x48x1x1xf32, 48x1x1x1>, %arg1: !migraphx.shaped<2x64x10x10xi8, 6400x100x10x1>,
                               %arg2: !migraphx.shaped<48x64x3x3xi8, 576x9x3x1>) -> !migraphx.shaped<2x48x10x10xi8, 4800x100x10x1> attributes {arch = "sm_100a", kernel = "mixr"} {
    %0 = migraphx.literal (dense<-5> : tensor<1xi8>) : <1xi8, 0>
    %1 = migraphx.literal (dense<2.500000e-01> : tensor<1xf32>) : <1xf32, 0>
    %2 = migraphx.literal (dense<1.22070313E-4> : tensor<1xf32>) : <1xf32, 0>
    %5 = migraphx.multibroadcast %0 {out_dyn_dims = [], out_lens = [2, 48, 10, 10]} : <1xi8, 0> -> <2x48x10x10xi8, 0x0x0x0>
    %6 = migraphx.multibroadcast %1 {out_dyn_dims = [], out_lens = [2, 48, 10, 10]} : <1xf32, 0> -> <2x48x10x10xf32, 0x0x0x0>
    %7 = migraphx.multibroadcast %2 {out_dyn_dims = [], out_lens = [2, 48, 10, 10]} : <1xf32, 0> -> <2x48x10x10xf32, 0x0x0x0>
    %8 = migraphx.quant_convolution %arg1, %arg2 {dilation = [1, 1], group = 1 : i64, padding = [1, 1, 1, 1], padding_mode = 0 : i64, stride = [1, 1]} : <2x64x10x10xi8, 6400x100x10x1>, <48x64x3x3xi8, 576x9x3x1> -> <2x48x10x10xi32, 4800x100x10x1>
    %9 = migraphx.dequantizelinear %8, %7 : <2x48x10x10xi32, 4800x100x10x1>, <2x48x10x10xf32, 0x0x0x0> -> <2x48x10x10xf32, 4800x100x10x1>
    %10 = migraphx.add %9, %arg0 : <2x48x10x10xf32, 4800x100x10x1>, <1x48x1x1xf32, 48x1x1x1> -> <2x48x10x10xf32, 4800x100x10x1>
    %11 = migraphx.relu %10 : <2x48x10x10xf32, 4800x100x10x1> -> <2x48x10x10xf32, 4800x100x10x1>
    %12 = migraphx.quantizelinear %11, %6, %5 : <2x48x10x10xf32, 4800x100x10x1>, <2x48x10x10xf32, 0x0x0x0>, !migraphx.shaped<2x48x10x10xi8, 0x0x0x0> -> <2x48x10x10xi8, 4800x100x10x1>
    return %12 : !migraphx.shaped<2x48x10x10xi8, 4800x100x10x1>
  }
}
"""


@pytest.fixture(scope="module")
def built():
    from rocmlir_b200 import _lib, build
    if not os.path.exists(_lib.LIB_PATH):
        build.build()
    return _lib.LIB_PATH


def test_c_client_runs_the_reference_call_sequence(built, tmp_path):
    exe = str(tmp_path / "mlirc_client")
    libdir = os.path.dirname(built)
    subprocess.run(["gcc", "-O1", "-I", os.path.join(ROOT, "include"), "-o", exe, os.path.join(ROOT, "tests", "mlirc_client.c"),
                    "-L", libdir, "-l:librocmlir_b200.so", f"-Wl,-rpath,{libdir}"], check=True)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    out = r.stdout
    assert r.returncode == 0 and "PASSED!" in out, out + r.stderr
    # the blob of mlirGetKernelInfo: the reference's own expectation for this graph (mlir/test/CAPI/mixr_cobj.cc:225-229)
    assert "4:<1,64,56,56> 4:<64,64,1,1> 1:<64> 4:<1,64,56,56>" in out
    assert "kernel name : main" in out
    assert "fails to update table, existing config is faster" in out       # the second, slower entry is rejected
    assert "block size : 256" in out and "magic 7f ELF" in out
    # the problem key has the reference's text format (mlir/test/rocmlir-gen/problem-key.mlir)
    assert "conv -F 1 -f GNC01 -I NGC01 -O NGC01 -n 1 -c 64 -H 56 -W 56 -k 64 -y 1 -x 1 -p 0 -q 0 -u 1 -v 1 -l 1 -j 1 -g 1" in out


def test_text_front_end_and_pipelines(built):
    from rocmlir_b200.mlirc import Module
    with Module(DOT_ADD) as m:
        m.high_level()
        assert m.kernel_info() == ([[1, 5, 4], [1, 4, 3], [1, 5, 3], [1, 5, 3]], "dot_add")
        assert m.key.endswith("-t f32 -out_datatype f32 -transA false -transB false -g 1 -m 5 -n 3 -k 4")
        with pytest.raises(Exception):
            m.binary()                       # nothing compiled yet
        m.backend("sm_100a")
        block, grid = m.kernel_attrs()
        assert block == 256 and grid >= 1
        assert m.binary()[:4] == b"\x7fELF"
    with Module(DOT_TRANSB_BIAS_RELU) as m:
        m.high_level()
        assert "-transA false -transB true -g 2 -m 384 -n 520 -k 256" in m.key
        # dims are reported in memory order: the column-major B [2][256][520] lies as [2][520][256]
        assert m.kernel_info() == ([[2, 384, 256], [2, 520, 256], [520], [2, 384, 520]], "mlir_dot_add_relu")
        assert m.set_perf_config("v2:128,128,8,64,64,8,1,1,1") and not m.set_perf_config("v2:nonsense")
        m.applicability()
        m.backend()
    with Module(CONV_BIAS_CLIP_NHWC) as m:
        m.high_level()
        assert "-f GN01C -I N01GC -O N01GC" in m.key                                  # KYXC filter, NHWC tensors
        args, name = m.kernel_info()
        assert args == [[1, 96, 1, 1], [2, 14, 14, 64], [96, 3, 3, 64], [2, 14, 14, 96]] and name == "mlir_convolution_add_clip"
        m.backend()
        assert m.workspace_size == 0         # implicit GEMM with the fused tail: one kernel, no scratch
    with Module(QUANT_CONV) as m:
        m.high_level()
        args, name = m.kernel_info()
        assert args[-1] == [2, 48, 10, 10] and name == "mlir_quantization"
        m.backend()


def test_what_cannot_be_fused_fails_the_pipeline_not_the_process(built):
    from rocmlir_b200.mlirc import Module, PipelineError
    bad_op = DOT_ADD.replace("migraphx.add %0, %arg2 {}", "migraphx.pow %0, %arg2")
    with Module(bad_op) as m:
        with pytest.raises(PipelineError, match="pow"):
            m.high_level()
    two = DOT_ADD.replace("return %2", "%9 = migraphx.dot %arg0, %arg1 : <1x5x4xf32, 20x4x1>, <1x4x3xf32, 12x3x1> -> <1x5x3xf32, 15x3x1>\n    return %2")
    with Module(two) as m:
        with pytest.raises(PipelineError, match="more than one contraction"):
            m.high_level()
    relu_before_add = DOT_TRANSB_BIAS_RELU.replace("migraphx.add %0, %1", "migraphx.add %r, %1").replace(
        "%1 = migraphx.multibroadcast", "%r = migraphx.relu %0 : <2x384x520xf16, 199680x520x1> -> <2x384x520xf16, 199680x520x1>\n  %1 = migraphx.multibroadcast").replace(
        "%3 = migraphx.relu %2", "%3 = migraphx.convert %2")
    with Module(relu_before_add) as m:
        with pytest.raises(PipelineError, match="fixed order"):
            m.high_level()
    with Module(DOT_ADD) as m:
        m.high_level()
        with pytest.raises(PipelineError):
            m.backend("gfx942")              # an AMD architecture name: mlirMIGraphXAddBackendPipeline answers false
    with pytest.raises(ValueError):
        Module("module { func.func @f(%a: !migraphx.shaped<4xf32, 1> -> oops }")
    strided = DOT_ADD.replace("20x4x1>", "40x8x2>")
    with Module(strided) as m:
        with pytest.raises(PipelineError, match="dense"):
            m.high_level()


def _reference_root():
    r = os.environ.get("ROCMLIR_REFERENCE_DIR") or os.path.join(os.path.dirname(ROOT), "reference")
    return r if os.path.isdir(os.path.join(r, "mlir", "test", "fusion", "pr-e2e")) else None


@pytest.mark.skipif(_reference_root() is None, reason="no reference checkout beside the repository")
def test_parser_reads_the_references_own_fusion_tests(built):
    """Where the reference checkout is at hand: every MIGraphX-level file of its fusion end-to-end tests must parse
    (or be refused with a message), and the dot / convolution + elementwise ones must pass the high-level pipeline."""
    from rocmlir_b200.mlirc import Module, PipelineError
    root = _reference_root()
    files = sorted(glob.glob(os.path.join(root, "mlir", "test", "fusion", "pr-e2e", "**", "mixr-*.mlir"), recursive=True))
    assert len(files) > 20
    parsed = fused = 0
    must_fuse = {"mixr-gemm-add.e2e.mlir", "mixr-gemm-bcast-add.e2e.mlir", "mixr-conv-bias-clipped-relu.mlir", "mixr-bcast-add.e2e.mlir"}
    seen = set()
    for f in files:
        text = open(f).read().replace("##TOKEN_ARCH##", "sm_100a")
        try:
            m = Module(text)
        except ValueError:
            continue
        parsed += 1
        try:
            m.high_level()
            fused += 1
            seen.add(os.path.basename(f))
        except PipelineError:
            pass
        m.close()
    assert parsed >= len(files) * 0.6, (parsed, len(files))
    assert must_fuse <= seen, must_fuse - seen


CONV_1D = """
module {
  func.func @conv1d_bias(%x: !migraphx.shaped<4x64x100xf16, 6400x1x64>, %w: !migraphx.shaped<128x64x5xf16, 320x1x64>,
                         %bias: !migraphx.shaped<1x128x1xf16, 128x1x1>) -> !migraphx.shaped<4x128x50xf16, 6400x1x128> attributes {kernel, arch = "sm_100a"} {
    %0 = migraphx.convolution %x, %w {dilation = [1], group = 1 : i64, padding = [2, 2], padding_mode = 0 : i64, stride = [2]} : <4x64x100xf16, 6400x1x64>, <128x64x5xf16, 320x1x64> -> <4x128x50xf16, 6400x1x128>
    %1 = migraphx.add %0, %bias : <4x128x50xf16, 6400x1x128>, <1x128x1xf16, 128x1x1> -> <4x128x50xf16, 6400x1x128>
    %2 = migraphx.relu %1 : <4x128x50xf16, 6400x1x128> -> <4x128x50xf16, 6400x1x128>
    return %2 : !migraphx.shaped<4x128x50xf16, 6400x1x128>
  }
}
"""


def test_one_dimensional_convolution_is_the_unit_height_problem(built):
    """A convolution over rank-3 tensors (n, c, w) is matched as the 2-D problem with a unit image height, the way
    MIGraphX itself expands it (mlir/lib/Conversion/MIGraphXToTosa/MIGraphXToTosa.cpp:241-275); here channels-last."""
    from rocmlir_b200.mlirc import Module
    with Module(CONV_1D) as m:
        m.high_level()
        key = m.key
        assert "convfp16 -F 1" in key and "-n 4 -c 64 -H 1 -W 100 -k 128 -y 1 -x 5 -p 0 -q 2 -u 1 -v 2 -l 1 -j 1 -g 1" in key
        assert "-I N01GC" in key or "-I N01C" in key or "-I NHWC" in key.upper(), key
        m.backend("sm_100a")
        assert m.binary()[:4] == b"\x7fELF"


DOT_SHARED_B = """
func.func @dot_shared_b(%a: !migraphx.shaped<8x96x64xf16, 6144x64x1>, %b: !migraphx.shaped<64x80xf16, 80x1>) -> !migraphx.shaped<8x96x80xf16, 7680x80x1> attributes {kernel, arch = "sm_100a"} {
  %0 = migraphx.multibroadcast %b {out_dyn_dims = [], out_lens = [8, 64, 80]} : <64x80xf16, 80x1> -> <8x64x80xf16, 0x80x1>
  %1 = migraphx.dot %a, %0 : <8x96x64xf16, 6144x64x1>, <8x64x80xf16, 0x80x1> -> <8x96x80xf16, 7680x80x1>
  return %1 : !migraphx.shaped<8x96x80xf16, 7680x80x1>
}
"""


def test_batched_dot_with_a_shared_second_operand_folds_the_batch_into_m(built):
    """A B operand broadcast along the batch (stride 0) makes G x M x K . K x N the (G M) x K . K x N product on the same
    bytes: one group of 768 rows instead of 8 groups of 96."""
    from rocmlir_b200.mlirc import Module, PipelineError
    with Module(DOT_SHARED_B) as m:
        m.high_level()
        assert "-transA false -transB false -g 1 -m 768 -n 80 -k 64" in m.key
    col_major_a = DOT_SHARED_B.replace("8x96x64xf16, 6144x64x1", "8x96x64xf16, 6144x1x96")
    with Module(col_major_a) as m:
        with pytest.raises(PipelineError, match="row-major first operand"):
            m.high_level()


# the shape of mlir/test/fusion/pr-e2e/mixr-dot-int4-f16.mlir at a size the tensor core sees: packed int4 weights as the
# first operand, unpacked along the reduction dimension and dequantised with a literal scale, then dot
DOT_INT4 = """
func.func @mlir_unpack_dequantizelinear_dot(%arg0: !migraphx.shaped<1x96x64xi8, 6144x64x1>, %arg1: !migraphx.shaped<1x128x80xf16, 10240x80x1>) -> !migraphx.shaped<1x96x80xf16, 7680x80x1> attributes {kernel, arch = "sm_100a"} {
  %0 = migraphx.literal (dense<[0.25]> : tensor<1xf16>) : <1xf16, 0>
  %1 = migraphx.multibroadcast %0 {out_dyn_dims = [], out_lens = [1, 96, 128]} : <1xf16, 0> -> <1x96x128xf16, 0x0x0>
  %2 = migraphx.unpack %arg0 {axis = 2 : i64, isUnsigned = false} : <1x96x64xi8, 6144x64x1> -> <1x96x128xi8, 12288x128x1>
  %3 = migraphx.dequantizelinear %2, %1 : <1x96x128xi8, 12288x128x1>, <1x96x128xf16, 0x0x0> -> <1x96x128xf16, 12288x128x1>
  %4 = migraphx.dot %3, %arg1 : <1x96x128xf16, 12288x128x1>, <1x128x80xf16, 10240x80x1> -> <1x96x80xf16, 7680x80x1>
  return %4 : !migraphx.shaped<1x96x80xf16, 7680x80x1>
}
"""


def test_int4_operand_is_unpacked_into_the_workspace(built):
    from rocmlir_b200.mlirc import Module, PipelineError
    with Module(DOT_INT4) as m:
        m.high_level()
        assert "-t f16 -out_datatype f16 -transA false -transB false -g 1 -m 96 -n 80 -k 128" in m.key
        assert m.kernel_info()[0][0] == [1, 96, 64]          # the kernel's first argument is still the packed tensor
        assert m.workspace_size >= 96 * 128 * 2              # room for the unpacked, dequantised operand
    along_rows = DOT_INT4.replace("axis = 2 : i64", "axis = 1 : i64")
    with Module(along_rows) as m:
        with pytest.raises(PipelineError, match="last, contiguous dimension"):
            m.high_level()


def test_unary_elementwise_ops_join_the_fused_tail(built):
    """dot -> add -> sigmoid (and the other unary ops of MIGraphX.td:134-181) are matched into the epilogue; two of them
    in a row, or one after the rectifier, are refused by the fixed order."""
    from rocmlir_b200.mlirc import Module, PipelineError
    text = DOT_TRANSB_BIAS_RELU.replace("migraphx.relu", "migraphx.sigmoid")
    with Module(text) as m:
        m.high_level()
        m.backend("sm_100a")
    twice = DOT_TRANSB_BIAS_RELU.replace("%3 = migraphx.relu %2", "%9 = migraphx.tanh %2 : <2x384x520xf16, 199680x520x1> -> <2x384x520xf16, 199680x520x1>\n  %3 = migraphx.erf %9")
    with Module(twice) as m:
        with pytest.raises(PipelineError, match="fixed order"):
            m.high_level()
