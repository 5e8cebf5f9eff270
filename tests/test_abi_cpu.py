"""The C-ABI library builds for sm_100a, loads on a machine without a GPU and exports
every symbol include/heddle_b200.h declares.  No compute call is made here."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def _declared_symbols():
    text = (ROOT / "include" / "heddle_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hb_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(built_lib):
    from heddle_b200 import _lib
    declared = _declared_symbols()
    assert declared, "no declarations found in the header"
    assert sorted(_lib.EXPORTS) == declared
    for name in declared:
        assert hasattr(built_lib, name), name


def test_version_and_static_queries(built_lib):
    from heddle_b200 import _lib
    assert built_lib.hb_version() == 100
    fa_smem = built_lib.hb_query(_lib.HB_QUERY_FA_SMEM)
    assert 0 < fa_smem <= 227 * 1024


def test_struct_layout_matches_header(built_lib):
    """ctypes mirrors of the argument structs have the C compiler's layout."""
    import subprocess, sys, tempfile
    from heddle_b200 import _lib
    src = r'''
#include <stdio.h>
#include <stddef.h>
#include "heddle_b200.h"
int main(void) {
  printf("%zu %zu %zu %zu\n", sizeof(hb_fa_args), offsetof(hb_fa_args, causal), offsetof(hb_fa_args, stream),
         offsetof(hb_fa_args, q_stride_b));
  printf("%zu %zu %zu\n", sizeof(hb_gemm_args), offsetof(hb_gemm_args, row_scale), offsetof(hb_gemm_args, stream));
  printf("%zu %zu\n", sizeof(hb_h2o_args), offsetof(hb_h2o_args, stream));
  printf("%zu %zu %zu %zu\n", sizeof(hb_prepare_args), offsetof(hb_prepare_args, ld_src), offsetof(hb_prepare_args, gamma),
         offsetof(hb_prepare_args, stream));
  printf("%zu %zu %zu %zu %zu\n", sizeof(hb_fa_bwd_args), offsetof(hb_fa_bwd_args, B), offsetof(hb_fa_bwd_args, q_stride_b),
         offsetof(hb_fa_bwd_args, causal), offsetof(hb_fa_bwd_args, stream));
  printf("%zu %zu %zu %zu\n", offsetof(hb_gemm_args, batch), offsetof(hb_gemm_args, w_layout), offsetof(hb_gemm_args, r_batch_stride),
         offsetof(hb_gemm_args, schedule));
  printf("%zu %zu %zu %zu %zu %zu %zu\n", sizeof(hb_rowwise_args), offsetof(hb_rowwise_args, rowscalar), offsetof(hb_rowwise_args, n_inputs),
         offsetof(hb_rowwise_args, rows), offsetof(hb_rowwise_args, program), offsetof(hb_rowwise_args, stream),
         offsetof(hb_rowwise_args, mode));
  return 0;
}'''
    with tempfile.TemporaryDirectory() as d:
        c = Path(d) / "t.c"
        c.write_text(src)
        exe = Path(d) / "t"
        subprocess.run(["gcc", "-std=c99", "-I", str(ROOT / "include"), str(c), "-o", str(exe)], check=True)
        lines = subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split("\n")
    fa = [int(x) for x in lines[0].split()]
    assert fa == [ctypes.sizeof(_lib.FaArgs), _lib.FaArgs.causal.offset, _lib.FaArgs.stream.offset,
                  _lib.FaArgs.q_stride_b.offset]
    gm = [int(x) for x in lines[1].split()]
    assert gm == [ctypes.sizeof(_lib.GemmArgs), _lib.GemmArgs.row_scale.offset, _lib.GemmArgs.stream.offset]
    h2 = [int(x) for x in lines[2].split()]
    assert h2 == [ctypes.sizeof(_lib.H2oArgs), _lib.H2oArgs.stream.offset]
    pw = [int(x) for x in lines[3].split()]
    assert pw == [ctypes.sizeof(_lib.PrepareArgs), _lib.PrepareArgs.ld_src.offset, _lib.PrepareArgs.gamma.offset,
                  _lib.PrepareArgs.stream.offset]
    bw = [int(x) for x in lines[4].split()]
    assert bw == [ctypes.sizeof(_lib.FaBwdArgs), _lib.FaBwdArgs.B.offset, _lib.FaBwdArgs.q_stride_b.offset,
                  _lib.FaBwdArgs.causal.offset, _lib.FaBwdArgs.stream.offset]
    gb = [int(x) for x in lines[5].split()]
    assert gb == [_lib.GemmArgs.batch.offset, _lib.GemmArgs.w_layout.offset, _lib.GemmArgs.r_batch_stride.offset,
                  _lib.GemmArgs.schedule.offset]
    rw = [int(x) for x in lines[6].split()]
    assert rw == [ctypes.sizeof(_lib.RowwiseArgs), _lib.RowwiseArgs.rowscalar.offset, _lib.RowwiseArgs.n_inputs.offset,
                  _lib.RowwiseArgs.rows.offset, _lib.RowwiseArgs.program.offset, _lib.RowwiseArgs.stream.offset,
                  _lib.RowwiseArgs.mode.offset]
    assert ctypes.sizeof(_lib.EwInst) == 16


def test_argument_validation_needs_no_gpu(built_lib):
    """Checks that run before any CUDA call return error codes with a message."""
    from heddle_b200 import _lib
    assert built_lib.hb_fa_fwd(None) == _lib.HB_ERR_BAD_ARG
    assert b"NULL" in built_lib.hb_last_error()
    a = _lib.FaArgs()
    a.B, a.Hq, a.Hkv, a.Sq, a.Skv, a.D = 1, 6, 4, 128, 128, 128
    assert built_lib.hb_fa_fwd(ctypes.byref(a)) == _lib.HB_ERR_BAD_ARG  # Hq % Hkv
    a.Hq = 4
    a.D = 96
    assert built_lib.hb_fa_fwd(ctypes.byref(a)) == _lib.HB_ERR_UNSUPPORTED
    assert b"head_dim" in built_lib.hb_last_error()
    a.D = 128
    a.Skv = 64
    a.causal = 1
    assert built_lib.hb_fa_fwd(ctypes.byref(a)) == _lib.HB_ERR_UNSUPPORTED  # causal with Skv < Sq
    a.causal = 0
    a.Skv = 0
    assert built_lib.hb_fa_fwd(ctypes.byref(a)) == _lib.HB_ERR_BAD_ARG
    a.Skv = 128
    assert built_lib.hb_fa_fwd(ctypes.byref(a)) == _lib.HB_ERR_BAD_ARG  # null pointers
    a.Sq = 0
    assert built_lib.hb_fa_fwd(ctypes.byref(a)) == _lib.HB_OK  # empty problem is a no-op
    for fn in (built_lib.hb_fa_bwd_preprocess, built_lib.hb_fa_bwd_dkdv, built_lib.hb_fa_bwd_dq):
        assert fn(None) == _lib.HB_ERR_BAD_ARG
        g = _lib.FaBwdArgs()
        g.B, g.Hq, g.Hkv, g.Sq, g.Skv, g.D, g.dtype = 1, 4, 4, 128, 128, 96, _lib.HB_BF16
        assert fn(ctypes.byref(g)) == _lib.HB_ERR_UNSUPPORTED  # head_dim 64 or 128
        assert b"head_dim" in built_lib.hb_last_error()
        g.D, g.dtype = 128, _lib.HB_FP8_E4M3
        assert fn(ctypes.byref(g)) == _lib.HB_ERR_UNSUPPORTED  # 16-bit types only
        g.dtype = _lib.HB_BF16
        assert fn(ctypes.byref(g)) == _lib.HB_ERR_BAD_ARG  # null pointers
        g.B = 0
        assert fn(ctypes.byref(g)) == _lib.HB_OK  # empty problem is a no-op
    assert built_lib.hb_prepare_weight(None) == _lib.HB_ERR_BAD_ARG
    w = _lib.PrepareArgs()
    w.n_src, w.K, w.dtype = 5, 64, _lib.HB_BF16
    assert built_lib.hb_prepare_weight(ctypes.byref(w)) == _lib.HB_ERR_BAD_ARG  # at most four matrices
    w.n_src, w.K = 1, 60
    assert built_lib.hb_prepare_weight(ctypes.byref(w)) == _lib.HB_ERR_ALIGN  # K % 8
    w.K = 64
    assert built_lib.hb_prepare_weight(ctypes.byref(w)) == _lib.HB_ERR_BAD_ARG  # null output
    # the rowwise program is checked on the host before anything is launched
    assert built_lib.hb_rowwise_program(None) == _lib.HB_ERR_BAD_ARG
    r = _lib.RowwiseArgs()
    r.rows, r.cols, r.dtype, r.n_outputs, r.n_inst = 4, 60, _lib.HB_BF16, 1, 1
    assert built_lib.hb_rowwise_program(ctypes.byref(r)) == _lib.HB_ERR_UNSUPPORTED  # cols % 8
    r.cols = 64
    assert built_lib.hb_rowwise_program(ctypes.byref(r)) == _lib.HB_ERR_ALIGN  # null output pointer
    buf = (ctypes.c_uint8 * 4096)()
    base = (ctypes.addressof(buf) + 15) & ~15
    r.outputs[0], r.ld_out[0] = base, 64
    r.program[0].op = _lib.EW_OPS["add"]
    r.program[0].src = _lib.EW_SRCS["imm"]
    assert built_lib.hb_rowwise_program(ctypes.byref(r)) == _lib.HB_ERR_BAD_ARG
    assert b"before a LOAD" in built_lib.hb_last_error()
    r.program[0].op = _lib.EW_OPS["load"]
    assert built_lib.hb_rowwise_program(ctypes.byref(r)) == _lib.HB_ERR_BAD_ARG
    assert b"never stored" in built_lib.hb_last_error()
    r.n_inst = 2
    r.program[1].op, r.program[1].src, r.program[1].index = _lib.EW_OPS["add"], _lib.EW_SRCS["tmp"], 1
    assert built_lib.hb_rowwise_program(ctypes.byref(r)) == _lib.HB_ERR_BAD_ARG
    assert b"before it is stored" in built_lib.hb_last_error()
    r.mode = 7
    assert built_lib.hb_rowwise_program(ctypes.byref(r)) == _lib.HB_ERR_BAD_ARG
    assert b"unknown mode" in built_lib.hb_last_error()


def _rowwise_args(program, cols=4096, dtype=None, n_in=2, n_vec=1, n_sc=1, n_out=1):
    """Arguments with aligned placeholder addresses: the compile-only hook never dereferences them."""
    from heddle_b200 import _lib
    a = _lib.RowwiseArgs()
    for i in range(n_in):
        a.inputs[i], a.ld_in[i] = 0x10000, cols
    for i in range(n_vec):
        a.rowvec[i] = 0x10000
    for i in range(n_sc):
        a.rowscalar[i] = 0x10000
    for i in range(n_out):
        a.outputs[i], a.ld_out[i] = 0x10000, cols
    a.n_inputs, a.n_rowvec, a.n_rowscalar, a.n_outputs = n_in, n_vec, n_sc, n_out
    a.rows, a.cols, a.dtype, a.n_inst = 128, cols, _lib.HB_BF16 if dtype is None else dtype, len(program)
    for pc, (op, src, idx, imm) in enumerate(program):
        a.program[pc].op, a.program[pc].src = _lib.EW_OPS[op], _lib.EW_SRCS[src or "none"]
        a.program[pc].index, a.program[pc].imm = idx, imm
    return a


def test_every_program_shape_compiles_for_sm100a_without_a_gpu(built_lib):
    """The run-time specialised rowwise kernels: source generation + NVRTC for sm_100a need no device."""
    from heddle_b200 import _lib
    if not built_lib.hb_rowwise_compiler_available():
        pytest.skip("libnvrtc cannot be loaded in this process")
    unary = [k for k, v in _lib.EW_OPS.items() if 16 <= v <= 30]
    binary = [k for k, v in _lib.EW_OPS.items() if 1 <= v <= 9]
    prog = [("load", "input", 0, 0.0)] + [(u, None, 0, 0.0) for u in unary] + [("store_tmp", None, 1, 0.0)]
    srcs = [("input", 1), ("rowvec", 0), ("rowscalar", 0), ("imm", 0), ("tmp", 1)]
    prog += [(b,) + srcs[i % 5] + (float("inf") if i == 3 else 1.5,) for i, b in enumerate(binary)]
    prog.append(("store_out", None, 0, 0.0))
    text = ctypes.create_string_buffer(1 << 16)
    for dtype in (_lib.HB_BF16, _lib.HB_FP16):
        rc = built_lib.hb_debug_rowwise_compile(ctypes.byref(_rowwise_args(prog, dtype=dtype)), text, len(text))
        assert rc == _lib.HB_OK, built_lib.hb_last_error()
    src = text.value.decode()
    assert src.count("EACH(") >= len(unary) + len(binary) and "0x7f800000" in src  # the infinite immediate, bit-exact
    softmax = [("load", "input", 0, 0.0), ("reduce_max", None, 0, 0.0), ("sub", "reduced", 0, 0.0), ("exp", None, 0, 0.0),
               ("store_tmp", None, 0, 0.0), ("reduce_sum", None, 1, 0.0), ("load", "tmp", 0, 0.0), ("div", "reduced", 1, 0.0),
               ("store_out", None, 0, 0.0)]
    for cols in (512, 4096):  # one warp per row / one CTA per row
        rc = built_lib.hb_debug_rowwise_compile(ctypes.byref(_rowwise_args(softmax, cols=cols)), text, len(text))
        assert rc == _lib.HB_OK, built_lib.hb_last_error()
        assert f"#define HB_WARPS_PER_ROW {1 if cols <= 1024 else 4}" in text.value.decode()
    # the hook validates like the entry point
    bad = _rowwise_args([("exp", None, 0, 0.0), ("store_out", None, 0, 0.0)])
    assert built_lib.hb_debug_rowwise_compile(ctypes.byref(bad), None, 0) == _lib.HB_ERR_BAD_ARG


def test_ops_reject_cpu_tensors(built_lib):
    from heddle_b200 import ops
    q = torch.zeros(1, 1, 128, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ops.fa_fwd(q, q, q)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from heddle_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setenv("HEDDLE_B200_LIB", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="not found"):
        _lib.load()
