"""The tuning surface without a GPU: problem keys in the reference's text format, perf_config strings, tuning
spaces, the best-entry table and the split-K likelihood rule. Expected strings come from the reference's own
tests (mlir/test/rocmlir-gen/problem-key.mlir, mlir/test/CAPI/mixr_split_k.cpp:327-329) with the architecture
field replaced by this hardware's."""
import ctypes as C
import threading

import pytest

from rocmlir_b200 import _lib as L
from rocmlir_b200 import tuning

CONV = ("--operation conv --arch sm_100a --in_type fp16 --fil_type fp16 --out_type fp16 --fil_layout GNC01 "
        "--in_layout NGC01 --out_layout NGC01 --batchsize 256 --groupsize 1 --in_channels 64 --out_channels 64 "
        "--in_h 56 --in_w 56 --out_h 56 --out_w 56 --fil_h 3 --fil_w 3 --padding_h 1 --padding_w 1")


def test_attention_key_matches_the_reference_format():
    # problem-key.mlir CHECK_2 (after the arch and numCU fields)
    p = tuning.Problem("--operation attention --arch sm_100a -t f16 -g 4 -seq_len_q 256 -seq_len_k 512 -head_dim_qk 64 "
                       "-head_dim_v 64")
    arch, num_cu, flags = p.key.split("\t")
    assert (arch, num_cu) == ("sm_100a", "148")
    assert flags == ("-t f16 -transQ false -transK false -transV false -transO false -g 4 -seq_len_q 256 "
                     "-seq_len_k 512 -head_dim_qk 64 -head_dim_v 64")
    # problem-key.mlir CHECK_4: --num_cu shows up in the key
    p = tuning.Problem("--operation attention --arch sm_100a --num_cu 304 -t f16 -g 4 -seq_len_q 256 -seq_len_k 512 "
                       "-head_dim_qk 64 -head_dim_v 64")
    assert p.key.split("\t")[1] == "304"


def test_gemm_and_conv_keys():
    g = tuning.Problem("--operation gemm --arch sm_100a -t i8 -g 2 -m 2048 -n 11008 -k 4096 -transB true")
    assert g.key.split("\t")[2] == "-t i8 -out_datatype i32 -transA false -transB true -g 2 -m 2048 -n 11008 -k 4096"
    c = tuning.Problem(CONV)
    assert c.key.split("\t")[2] == ("convfp16 -F 1 -f GNC01 -I NGC01 -O NGC01 -n 256 -c 64 -H 56 -W 56 -k 64 -y 3 -x 3 "
                                     "-p 1 -q 1 -u 1 -v 1 -l 1 -j 1 -g 1")
    w = tuning.Problem(CONV.replace("--operation conv", "--operation conv_bwd_weight").replace("GNC01", "GN01C")
                       .replace("NGC01", "N01GC"))
    assert " -F 4 -f GN01C -I N01GC -O N01GC " in w.key
    # a key's flag text is itself a valid option string for the same problem
    again = tuning.Problem("--operation gemm --arch sm_100a " + g.key.split("\t")[2])
    assert again.key == g.key


def test_key_buffer_has_strncpy_semantics():
    lib = L.lib()
    p = tuning.Problem(CONV)
    full = p.key.encode()
    buf = C.create_string_buffer(b"\xff" * 16, 16)
    n = lib.rbTuningGetKey(p._p, buf, 8)
    assert n == len(full)                       # true length, whatever the buffer size
    assert buf.raw[:8] == full[:8] and buf.raw[8] == 0xff   # no terminator written, nothing past bufLen touched
    assert lib.rbTuningGetKey(L._Handle(None), buf, 8) == tuning.SIZE_MAX


def test_split_k_likelihood_examples_of_the_reference():
    assert tuning.is_split_k_faster(1, 1024, 1024, 64) == tuning.MAYBE
    assert tuning.is_split_k_faster(1, 8192, 8192, 64) == tuning.NEVER
    assert tuning.is_split_k_faster(1, 64, 64, 1024) == tuning.ALWAYS
    assert tuning.is_split_k_faster(1, 64, 64, 1024, level=tuning.QUICK) == tuning.NEVER   # the quick set never splits


def test_spaces_and_param_strings():
    p = tuning.Problem("--operation gemm --arch sm_100a -t f16 -m 4096 -n 4096 -k 4096")
    quick, full, exhaustive = p.space(tuning.QUICK), p.space(tuning.FULL), p.space(tuning.EXHAUSTIVE)
    assert quick[0] == "b200:256,256,0,1,0"                 # the library's own choice comes first
    assert 1 < len(quick) < len(full) < len(exhaustive)
    assert set(quick) <= set(full)
    assert p.quick_space() == quick                        # GetQuick on a full space
    assert len(set(full)) == len(full)
    for s in full:
        assert p.set_from_str(s), s
        assert p.perf_config == s
    # a skinny problem: tiles that would be at least half empty are not offered, K splits are
    skinny = tuning.Problem("--operation gemm --arch sm_100a -t f16 -m 64 -n 64 -k 8192")
    assert all(s.startswith("b200:128,64,") for s in skinny.space(tuning.FULL))
    assert any(int(s.split(",")[3]) > 1 for s in skinny.space(tuning.FULL))
    assert not skinny.set_from_str("b200:128,64,0,200,0")     # more K ranges than the library will make
    assert not p.set_from_str("b200:256,256,0,1")           # malformed
    assert not p.set_from_str("garbage")
    assert p.is_fusible("b200:256,256,0,4,0") and not p.is_fusible("nonsense")
    assert p.num_prefill_args == 0 and p.num_aux_buffers == 0


def test_table_keeps_the_fastest_entry_and_is_shareable():
    p = tuning.Problem("--operation gemm --arch sm_100a -t f16 -m 4096 -n 4096 -k 4096")
    t = tuning.Table()
    assert not p.set_from_table(t)                          # empty table
    assert t.update(p.key, "b200:256,128,0,1,0", 2.0)
    assert not t.update(p.key, "b200:128,128,0,1,0", 3.0)     # slower: rejected
    assert t.update(p.key, "b200:256,256,0,1,0", 1.0)         # faster: replaces
    assert p.set_from_table(t) and p.perf_config == "b200:256,256,0,1,0"
    other = tuning.Problem("--operation gemm --arch sm_100a -t f16 -m 512 -n 512 -k 512")
    assert not other.set_from_table(t)

    def writer(i):
        for j in range(200):
            t.update(f"key{j % 7}", "b200:256,256,0,1,0", float(1000 - i - j))
    threads = [threading.Thread(target=writer, args=(i,)) for i in range(4)]
    [th.start() for th in threads]
    [th.join() for th in threads]
    assert not t.update("key0", "b200:256,256,0,1,0", 5000.0)


def test_get_config_reports_the_launch():
    lib = L.lib()
    p = L.RbGemmProblem(1, 4096, 4096, 4096, 0, 0, 0, L.F16, L.F16, 0)
    info = L.RbGemmConfigInfo()
    assert lib.rbGemmGetConfig(C.byref(p), C.byref(info)) == L.SUCCESS
    assert (info.tile_m, info.tile_n, info.tile_k, info.ctas, info.splits) == (256, 256, 64, 2, 1)
    assert info.grid == 148 and info.block == 256 and 0 < info.dynamic_smem <= 232448
    # the explicit variant word reproduces the configuration
    lib.rbSetGemmVariant(info.variant)
    again = L.RbGemmConfigInfo()
    assert lib.rbGemmGetConfig(C.byref(p), C.byref(again)) == L.SUCCESS
    lib.rbSetGemmVariant(0)
    assert (again.tile_n, again.ctas, again.stages, again.splits) == (info.tile_n, info.ctas, info.stages, info.splits)
    assert lib.rbGetGemmVariant() == 0


def test_tuning_database_text_forms_and_lookup(tmp_path):
    """The tuning database in the reference's text forms (tuningRunner.py:393-404 writes 4 or 5 columns, perfRunner.py:
    174-200 also reads the legacy 3): a table round-trips through a file, the process-wide database takes the rows of
    this architecture and a launch with variant 0 then plans with the recorded configuration."""
    import ctypes as C
    from rocmlir_b200 import _lib as L
    opts = "--operation gemm --arch sm_100a --t f16 --out_datatype f16 --g 1 --m 4096 --n 4096 --k 4096 --transA false --transB false"
    prob = tuning.Problem(opts)
    key = prob.key
    assert key.split("\t")[:2] == ["sm_100a", "148"]
    table = tuning.Table()
    assert table.update(key, "b200:256,128,0,1,0", 2.0)
    assert table.update(key, "b200:128,256,0,1,0", 1.0)        # faster: replaces
    assert not table.update(key, "b200:128,64,0,1,0", 3.0)     # slower: kept out
    path = str(tmp_path / "db.tsv")
    assert table.save(path, "full") == 1
    lines = open(path).read().splitlines()
    assert lines[0].startswith("# arch\tnumCUs\ttestVector\tperfConfig")
    assert lines[1] == key + "\tb200:128,256,0,1,0"
    again = tuning.Table()
    assert again.load(path) == 1
    fresh = tuning.Problem(opts)
    assert fresh.set_from_table(again) and fresh.perf_config == "b200:128,256,0,1,0"
    # the three column counts, a comment, a foreign architecture, an unmappable string
    problem = key.split("\t", 2)[2]
    mixed = tmp_path / "mixed.tsv"
    mixed.write_text("# arch\tnumCUs\ttestVector\tperfConfig\tTFlops (full)\n"
                     f"sm_100a\t148\t{problem}\tb200:256,128,0,1,0\t1234.5\n"
                     f"gfx942\t304\t{problem}\tv2:64,64,16,32,32,4,1,1,1\t512.0\n"
                     f"sm_100a\t{problem.replace('-m 4096', '-m 2048')}\tb200:128,128,0,1,0\n"
                     f"sm_100a\t148\t{problem.replace('-m 4096', '-m 1024')}\tnot-a-config\n")
    saved = L.lib().rbGetGemmVariant()
    tuning.db_clear()
    try:
        assert tuning.db_load(str(mixed)) == 2 and tuning.db_size() == 2
        assert tuning.db_lookup(prob) == prob_variant("b200:256,128,0,1,0", opts)
        gp = prob_gemm(4096)
        info = L.RbGemmConfigInfo()
        L.lib().rbSetGemmVariant(0)
        assert L.lib().rbGemmGetConfig(C.byref(gp), C.byref(info)) == 0
        assert (info.ctas, info.tile_n) == (2, 128)                 # the recorded tile, not the rule's 256 columns
        L.lib().rbSetGemmVariant(prob_variant("b200:128,64,0,1,0", opts))
        assert L.lib().rbGemmGetConfig(C.byref(gp), C.byref(info)) == 0
        assert (info.ctas, info.tile_n) == (1, 64)                  # an explicit variant word wins over the database
        L.lib().rbSetGemmVariant(0)
        gp2 = prob_gemm(2048)                                   # the legacy 3-column row
        assert L.lib().rbGemmGetConfig(C.byref(gp2), C.byref(info)) == 0 and (info.ctas, info.tile_n) == (1, 128)
        tuning.db_clear()
        assert L.lib().rbGemmGetConfig(C.byref(gp), C.byref(info)) == 0 and info.tile_n == 256
    finally:
        tuning.db_clear()
        L.lib().rbSetGemmVariant(saved)


def prob_variant(perf, opts):
    q = tuning.Problem(opts)
    assert q.set_from_str(perf)
    return q.variant


def prob_gemm(m):
    from rocmlir_b200 import _lib as L
    gp = L.RbGemmProblem()
    gp.g, gp.m, gp.n, gp.k = 1, m, 4096, 4096
    gp.trans_a = gp.trans_b = gp.trans_c = 0
    gp.ab_type = gp.c_type = L.F16
    return gp
