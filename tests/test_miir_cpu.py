"""The string-configured handle API without a GPU: option grammar, validation, kernel count, workspace, the
lowering state machine and the two-call buffer protocol. Cases follow the reference's own tests of this API
(mlir/test/mlir-rock-lib/{populate_fw,populate_bwd,populate_bww,workspace,archname}.mlir and applicability/*.mlir)
with the architecture replaced by this hardware's name."""
import ctypes as C

import pytest

from rocmlir_b200 import _lib as L
from rocmlir_b200 import miir

BASE = (" --operation {op} --arch {arch} --num_cu 148 --in_type {t} --fil_type {t} --out_type {t} --fil_layout GNCHW "
        "--in_layout NGCHW --out_layout NGCHW --batchsize 64 --in_channels 1024 --out_channels 1024 --in_h 14 --in_w 14 "
        "--out_h 14 --out_w 14 --fil_h 1 --fil_w 1 --dilation_h 1 --dilation_w 1 --conv_stride_h 1 --conv_stride_w 1 "
        "--padding_h 0 --padding_w 0 --kernel_name conv_nchw_kcyx_nkhw --groupsize 1")


def opts(op="conv", arch="sm_100a", t="fp16", extra=""):
    return BASE.format(op=op, arch=arch, t=t) + " " + extra


@pytest.mark.parametrize("op", ["conv", "conv_bwd_data", "conv_bwd_weight"])
@pytest.mark.parametrize("t", ["fp32", "fp16", "bf16"])
def test_handle_for_every_direction_and_float_type(op, t):
    with miir.Handle(opts(op, t=t)) as h:
        assert h.kernel_count == 1            # the whole operation is one handle here
        assert h.workspace_size >= 0
        h.lower_tuning_params()
        g, l = h.execution_dims()
        assert l == 256 and g % l == 0 and 0 < g // l <= 148


def test_null_handle_conventions():
    lib = L.lib()
    assert lib.miirGetKernelCount(None) == -1          # rocmlir-lib.cpp:160-166
    assert lib.miirGetWorkspaceSize(None) == 0         # :168-174
    assert lib.miirDestroyHandle(None) == miir.INVALID_PARAM
    assert lib.miirLowerBin(None) == miir.INVALID_PARAM
    assert lib.miirLowerTuningParams(None) == miir.INVALID_PARAM
    g, l = C.c_size_t(), C.c_size_t()
    assert lib.miirGetExecutionDims(None, C.byref(g), C.byref(l)) == miir.INVALID_PARAM


@pytest.mark.parametrize("arch", ["amdgcn-amd-amdhsa:gfx908:sramecc+:xnack-", "amdgcn-amd-amdhsa:gfx906", "gfx942",
                                  "amdgcn-amd-amdhsa:aa", "sm_90a", ""])
def test_foreign_architectures_give_null(arch):
    with pytest.raises(ValueError):
        miir.Handle(opts(arch=arch))


def test_accepted_architecture_spellings():
    for arch in ("sm_100a", "sm_100", "nvptx64-nvidia-cuda:sm_100a"):
        miir.Handle(opts(arch=arch)).close()


@pytest.mark.parametrize("missing", ["batchsize", "groupsize", "in_layout", "in_type", "in_channels", "in_h", "in_w",
                                     "out_layout", "out_type", "out_channels", "out_h", "out_w", "fil_layout",
                                     "fil_type", "fil_w", "fil_h", "arch", "operation"])
def test_every_required_key_is_required(missing):
    toks = opts().split()
    i = toks.index("--" + missing)
    del toks[i:i + 2]
    with pytest.raises(ValueError):
        miir.Handle(" ".join(toks))


def test_inconsistent_dimensions_give_null():
    # output size that does not follow from input, filter, padding, stride and dilation (ConvGenerator.cpp:221-236)
    with pytest.raises(ValueError):
        miir.Handle(opts().replace("--out_h 14", "--out_h 13"))
    # input plus padding smaller than the filter (:238-245)
    bad = opts().replace("--fil_h 1", "--fil_h 17").replace("--out_h 14", "--out_h -2")
    with pytest.raises(ValueError):
        miir.Handle(bad)
    # channels not divisible by the group count
    with pytest.raises(ValueError):
        miir.Handle(opts().replace("--groupsize 1", "--groupsize 3"))
    # layouts of different length / repeated letters / 3-D
    with pytest.raises(ValueError):
        miir.Handle(opts().replace("--in_layout NGCHW", "--in_layout NGCH"))
    with pytest.raises(ValueError):
        miir.Handle(opts().replace("--in_layout NGCHW", "--in_layout NGCHH"))
    # a third image letter: accepted while every depth is 1 (the tensor is the 2-D tensor on the same bytes) ...
    three = opts().replace("NGCHW", "NGCHWD").replace("GNCHW", "GNCHWD")
    with miir.Handle(three) as h3, miir.Handle(opts()) as h2:
        assert h3.workspace_size == h2.workspace_size and h3.kernel_count == h2.kernel_count
    miir.Handle(three + " --in_d 1 --fil_d 1 --out_d 1").close()
    # ... a real depth has no kernel behind this option grammar (rbConv3d is the entry point for it)
    with pytest.raises(ValueError):
        miir.Handle(three + " --in_d 4 --fil_d 3 --out_d 2")
    with pytest.raises(ValueError):
        miir.Handle(opts().replace("NGCHW", "NGCHWD"))          # only one of the three layouts names the depth


def test_eight_bit_types_run_forward_only():
    # ConvGenerator.cpp:631-638
    i8 = opts(t="i8").replace("--out_type i8", "--out_type i32")
    miir.Handle(i8).close()
    for t in ("fp8", "bf8"):                   # 8-bit floats accumulate and store f32
        f8 = opts(t=t).replace(f"--out_type {t}", "--out_type fp32")
        miir.Handle(f8).close()
        with pytest.raises(ValueError):
            miir.Handle(opts(t=t))            # ... and nothing else
        for op in ("conv_bwd_data", "conv_bwd_weight"):
            with pytest.raises(ValueError):
                miir.Handle(f8.replace("--operation conv", "--operation " + op))
    for op in ("conv_bwd_data", "conv_bwd_weight"):
        with pytest.raises(ValueError):
            miir.Handle(i8.replace("--operation conv", "--operation " + op))
    with pytest.raises(ValueError):
        miir.Handle(opts(t="i8"))             # i8 x i8 stores i32


def test_layout_spellings_of_the_reference():
    # the four layout triples the reference enables (rocmlir-lib.cpp:94-113), upper or lower case, digits or letters
    triples = [("GNCHW", "NGCHW", "NGCHW"), ("GNHWC", "NHWGC", "NHWGC"), ("gnc01", "ngc01", "ngc01"),
               ("gn01c", "n01gc", "n01gc"), ("gkcyx", "ngchw", "ngkhw"), ("gkyxc", "nhwgc", "nhwgk")]
    for f, i, o in triples:
        s = opts().replace("--fil_layout GNCHW", "--fil_layout " + f).replace("--in_layout NGCHW", "--in_layout " + i)
        s = s.replace("--out_layout NGCHW", "--out_layout " + o)
        miir.Handle(s).close()


def test_kernel_id_and_duplicates():
    miir.Handle(opts(extra="--kernel_id 0")).close()
    with pytest.raises(ValueError):
        miir.Handle(opts(extra="--kernel_id 1"))
    # a later duplicate overwrites (std::map assignment in the reference's tokeniser)
    with miir.Handle(opts(extra="--batchsize 32")) as h:
        h.lower_tuning_params()
        g32, _ = h.execution_dims()
    with miir.Handle(opts()) as h:
        h.lower_tuning_params()
        g64, _ = h.execution_dims()
    assert g32 <= g64


def test_lowering_state_machine_and_buffer_protocol():
    lib = L.lib()
    with miir.Handle(opts("conv_bwd_weight")) as h:
        g, l = C.c_size_t(), C.c_size_t()
        assert lib.miirGetExecutionDims(h._h, C.byref(g), C.byref(l)) == miir.INVALID_MODULE   # nothing lowered yet
        size = C.c_size_t(0)
        assert lib.miirBufferGet(h._h, None, C.byref(size)) == miir.INVALID_MODULE
        assert lib.miirBufferGet(h._h, None, None) == miir.INVALID_PARAM                       # rocmlir-lib.cpp:296-297
        h.lower_tuning_params()
        assert lib.miirBufferGet(h._h, None, C.byref(size)) == miir.INVALID_MODULE             # tuned, but no binary
        h.lower_bin()
        # the code object is an ELF image (the sm_100a cubin), as the reference's is an ELF hsaco
        assert lib.miirBufferGet(h._h, None, C.byref(size)) == miir.SUCCESS and size.value > 1 << 20
        image = h.buffer()
        assert image[:4] == b"\x7fELF" and len(image) == size.value
        blob = h.descriptor()
        assert blob[:7] == b"RB2KDSC" and len(blob) > 64
        assert lib.miirGetExecutionDims(h._h, None, C.byref(l)) == miir.INVALID_PARAM
        # a descriptor with a damaged header is refused before anything is launched
        bad = b"XXXXXXXX" + blob[8:]
        assert lib.miirLaunchFromBuffer(bad, len(bad), None, None, None, None, None, 0, None) == miir.INVALID_MODULE
        assert lib.miirLaunchFromBuffer(blob, len(blob) - 1, None, None, None, None, None, 0, None) == miir.INVALID_PARAM


def test_perf_config_selects_the_tile():
    with miir.Handle(opts(extra="--perf_config b200:128,128,0,1,0")) as h:
        h.lower_tuning_params()
        g_small, _ = h.execution_dims()
    # the reference's own strings are accepted and mapped onto the nearest tile (MPerBlock <= 128: one CTA per tile;
    # NPerBlock 64 -> 64-column tiles), here the one of mlir/test/CAPI/mixr_split_k.cpp:351
    with miir.Handle(opts(extra="--perf_config v2:64,64,16,32,32,4,1,1,1")) as h:
        h.lower_tuning_params()
        g_ref, l_ref = h.execution_dims()
        assert l_ref == 256 and g_ref > 0
    with miir.Handle(opts(extra="--perf_config 128,128,8,64,64,8,1,1")) as h:      # version 1: un-prefixed, no split field
        h.lower_tuning_params()
    for bad in ("b200:100,128,0,1,0", "v2:64,64,16", "v2:64,64,16,32,32,4,0,1,1", "v2:64,x,16,32,32,4,1,1,1",
                "v2:512,64,16,32,32,4,1,1,1", "v1:128,128,0,1,0", "64,64,16,32,32,4,1,1,1,1"):
        with pytest.raises(ValueError):     # unmappable strings fail applicability (a NULL handle), they do not crash
            miir.Handle(opts(extra="--perf_config " + bad))
    assert g_small > 0


def test_gemm_and_attention_extensions():
    with miir.Handle("--operation gemm --arch sm_100a -t f16 -out_datatype f16 -transA false -transB true -g 1 "
                     "-m 4096 -n 4096 -k 4096") as h:
        h.lower_bin()
        g, l = h.execution_dims()
        assert (g // l, l) == (148, 256)
        assert h.workspace_size == 0
    with miir.Handle("--operation attention --arch sm_100a -t f16 -g 512 -seq_len_q 2048 -seq_len_k 2048 "
                     "-head_dim_qk 128 -head_dim_v 128 -transK true") as h:
        h.lower_tuning_params()
        g, l = h.execution_dims()
        assert g // l == 512 * 8
    with pytest.raises(ValueError):
        miir.Handle("--operation attention --arch sm_100a -t f32 -g 1 -seq_len_q 64 -seq_len_k 64 -head_dim_qk 64 "
                    "-head_dim_v 64")
    with pytest.raises(ValueError):
        miir.Handle("--operation gemm --arch sm_100a -t f16 -m 0 -n 8 -k 8")
