"""CPU-side checks: the C-ABI library loads, exports every symbol the header declares, and its
host-only logic (emitter selection, argument validation without a device) behaves."""
import ctypes as C
import os
import re

import pytest

from sanic_b200 import _abi as abi
from sanic_b200 import backend

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    text = open(os.path.join(ROOT, "include", "sanic_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sanic_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = abi.load()
    names = header_functions()
    assert len(names) >= 35
    for n in names:
        assert hasattr(lib, n), f"libsanic_b200.so does not export {n}"
        assert n in abi.PROTOTYPES, f"{n} has no ctypes prototype"
    assert set(abi.PROTOTYPES) == set(names)


def test_version_and_open_without_device():
    lib = abi.load()
    assert b"sm_100a" in lib.sanic_version()
    try:
        import torch
        if torch.cuda.is_available():
            pytest.skip("a device is present")
    except ImportError:
        pass
    h = C.c_void_p()
    assert lib.sanic_cuda_open(0, C.byref(h)) != abi.OK  # no silent CPU fallback
    assert not h.value


def _select(kinds, refs=None, leaf=abi.F32, body=False, defer=False):
    c = backend.make_carrier(kinds, refs, leaf, body, defer)
    fam = C.c_int32(-1)
    rc = abi.load().sanic_emit_select(C.byref(c), C.byref(fam))
    return rc, fam.value


def test_emitter_selects_by_carrier_structure():
    # the four derived carriers (reference tests/laws.rs:107-126,620-646; tests/compile.rs:139-171)
    A, MX, MN, ES, AE = abi.SLOT_PLAIN_ADD, abi.SLOT_PLAIN_MAX, abi.SLOT_PLAIN_MIN, abi.SLOT_EXP_SHIFTED, abi.SLOT_AT_EXTREMUM
    assert _select([MX, ES, ES], [0, 0, 0], abi.BF16, body=True) == (abi.OK, abi.KERNEL_ONLINE_SOFTMAX_FOLD)
    assert _select([A, A], [0, 0], abi.BF16, defer=True) == (abi.OK, abi.KERNEL_DEFERRED_NORM_CONTRACTION)
    assert _select([A], [0], abi.I4) == (abi.OK, abi.KERNEL_GROUPED_I4_CONTRACTION)
    assert _select([A], [0], abi.BF16) == (abi.OK, abi.KERNEL_PLAIN_CONTRACTION)
    assert _select([MX, AE], [0, 0]) == (abi.OK, abi.KERNEL_EXTREMUM_INDEX)
    # structures with no kernel are refused, not approximated
    assert _select([MN, ES, ES], [0, 0, 0], abi.BF16, body=True)[0] == abi.ERR_UNSUPPORTED
    assert _select([MX, ES, ES], [0, 1, 0], abi.BF16, body=True)[0] == abi.ERR_UNSUPPORTED
    assert _select([MX, MX])[0] == abi.ERR_UNSUPPORTED


def test_struct_sizes_match_the_header():
    # compile a probe with the same header and compare sizeof / a few offsets
    import subprocess
    import tempfile
    src = r'''
#include <stdio.h>
#include <stddef.h>
#include "sanic_b200.h"
int main(void) {
  printf("%zu %zu %zu %zu ", sizeof(sanic_fitted_specs), offsetof(sanic_fitted_specs, sm_count), sizeof(sanic_fold_plan), offsetof(sanic_fold_plan, seconds));
  printf("%zu %zu %zu %zu %zu %zu %zu %zu %zu %zu ", sizeof(sanic_buffer_decl), sizeof(sanic_reloc), sizeof(sanic_schedule_desc),
         sizeof(sanic_binding), sizeof(sanic_buffer_view), sizeof(sanic_state_decl), offsetof(sanic_stage_desc, u.embed.scales),
         offsetof(sanic_decode_params, kv_cap), offsetof(sanic_attn_params, accum_dtype), offsetof(sanic_peer_exchange, spin_limit));
  printf("%zu %zu %zu %zu ", offsetof(sanic_stage_desc, u.attn.storage), offsetof(sanic_stage_desc, u.attn.p.mask),
         offsetof(sanic_stage_desc, u.gemm.y), offsetof(sanic_stage_desc, u.rope.table));
  printf("%zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu\n", sizeof(sanic_device_specs), sizeof(sanic_carrier_desc),
         sizeof(sanic_attn_params), sizeof(sanic_decode_params), sizeof(sanic_gemm_rmsnorm_params),
         sizeof(sanic_gemv_params), sizeof(sanic_rope_cache_params), sizeof(sanic_stage_desc),
         offsetof(sanic_stage_desc, u), sizeof(sanic_peer_exchange), offsetof(sanic_peer_exchange, epoch),
         sizeof(sanic_expr_op), sizeof(sanic_operand), offsetof(sanic_operand, gather_extent), sizeof(sanic_generic_desc),
         offsetof(sanic_generic_desc, project), offsetof(sanic_generic_desc, out_dtype));
  return 0; }
'''
    with tempfile.TemporaryDirectory() as d:
        c = os.path.join(d, "p.c")
        open(c, "w").write(src)
        exe = os.path.join(d, "p")
        subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), c, "-o", exe], check=True)
        got = [int(t) for t in subprocess.run([exe], capture_output=True, text=True, check=True).stdout.split()]
    want = [C.sizeof(abi.FittedSpecs), abi.FittedSpecs.sm_count.offset, C.sizeof(abi.FoldPlan), abi.FoldPlan.seconds.offset,
            C.sizeof(abi.BufferDecl), C.sizeof(abi.Reloc), C.sizeof(abi.ScheduleDesc), C.sizeof(abi.Binding), C.sizeof(abi.BufferView),
            C.sizeof(abi.StateDecl), abi.StageDesc.u.offset + abi._StageUnion.embed.offset + abi._EmbedStage.scales.offset,
            abi.DecodeParams.kv_cap.offset, abi.AttnParams.accum_dtype.offset, abi.PeerExchange.spin_limit.offset,
            abi.StageDesc.u.offset + abi._StageUnion.attn.offset + abi._AttnStage.storage.offset,
            abi.StageDesc.u.offset + abi._StageUnion.attn.offset + abi.AttnParams.mask.offset,
            abi.StageDesc.u.offset + abi._StageUnion.gemm.offset + abi.GemmRmsnormParams.y.offset,
            abi.StageDesc.u.offset + abi._StageUnion.rope.offset + abi._RopeStage.table.offset,
            C.sizeof(abi.DeviceSpecs), C.sizeof(abi.CarrierDesc), C.sizeof(abi.AttnParams), C.sizeof(abi.DecodeParams),
            C.sizeof(abi.GemmRmsnormParams), C.sizeof(abi.GemvParams), C.sizeof(abi.RopeCacheParams),
            C.sizeof(abi.StageDesc), abi.StageDesc.u.offset, C.sizeof(abi.PeerExchange), abi.PeerExchange.epoch.offset,
            C.sizeof(abi.ExprOp), C.sizeof(abi.Operand), abi.Operand.gather_extent.offset, C.sizeof(abi.GenericDesc),
            abi.GenericDesc.project.offset, abi.GenericDesc.out_dtype.offset]
    assert got == want


def test_device_class_refuses_to_run_without_cuda():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    with pytest.raises(backend.RunError):
        backend.CudaDevice(0)
