"""CPU-only checks: the C-ABI library loads and exports what include/rglru_b200.h declares, argument
validation returns the documented status codes (these paths return before any CUDA call), and the
host-side module layer mirrors the reference's error behaviour."""

from __future__ import annotations

import ctypes
import os
import re

import pytest
import torch

from conftest import ROOT, load_golden, params_of

HEADER = os.path.join(ROOT, "include", "rglru_b200.h")


@pytest.fixture(scope="module")
def lib():
    from griffin_b200 import _lib
    from griffin_b200.build import build_library
    build_library()
    return _lib.load()


def _declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rglru_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(lib):
    from griffin_b200 import _lib
    names = _declared_functions()
    assert len(names) >= 15
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for name in names:
        assert hasattr(raw, name), f"{name} is declared in the header but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert lib.rglru_abi_version() == 2


def test_status_strings(lib):
    texts = {lib.rglru_status_string(code).decode() for code in range(9)}
    assert len(texts) == 9 and "ok" in texts
    assert lib.rglru_status_string(1234).decode() == "unknown status"


def test_workspace_size_and_chunk(lib):
    from griffin_b200 import _lib
    chunk = lib.rglru_chunk_steps(_lib.BF16)
    assert chunk > 0 and chunk % 16 == 0
    B, T, D = 3, 130, 40
    nsave = -(-T // chunk)
    # chunk-entry states, per-row dLambda partials, a 256-byte tail holding the completion ticket, per-row gate sums
    assert lib.rglru_workspace_bytes(B, T, D, _lib.F32) == 4 * (B * nsave * D + B * D) + 256 + 4 * B * 2 * D
    assert lib.rglru_workspace_bytes(0, T, D, _lib.F32) == 0
    assert lib.rglru_conv_bwd_workspace_bytes(B, T, D) >= 4 * 5 * D * B
    # the arithmetic that shape inference (the ops' fake implementations) uses is the library's own
    from griffin_b200.ops import workspace_bytes
    for shape in ((3, 130, 40), (8, 2048, 1024), (1, 1, 1), (64, 8192, 5632)):
        assert workspace_bytes(*shape) == lib.rglru_workspace_bytes(*shape, _lib.BF16)


def test_argument_validation_codes(lib):
    """Every check below is made before the library touches the CUDA runtime."""
    from griffin_b200 import _lib
    buf = (ctypes.c_float * 64)()
    p = ctypes.addressof(buf)
    ok_args = dict(B=1, T=2, D=4)
    # dtype
    assert lib.rglru_fwd(p, p, p, p, None, None, p, None, None, 0, 1, 2, 4, 8.0, 7, None) == _lib.ERR_BAD_DTYPE
    # null pointers
    assert lib.rglru_fwd(None, p, p, p, None, None, p, None, None, 0, 1, 2, 4, 8.0, _lib.F32, None) == _lib.ERR_NULL_POINTER
    assert lib.rglru_bwd(p, None, p, p, p, p, None, None, p, 1 << 20, p, p, None, p, None, 1, 2, 4, 8.0, _lib.F32, None) == _lib.ERR_NULL_POINTER
    # carry-only forms: rglru_fwd itself needs y; the backward takes all four gradient outputs absent plus dh0, or none absent
    assert lib.rglru_fwd(p, p, p, p, None, None, None, p, None, 0, 1, 2, 4, 8.0, _lib.F32, None) == _lib.ERR_NULL_POINTER
    assert lib.rglru_fwd_carry(p, p, p, p, None, None, None, p, None, None, 0, 1, 2, 4, 8.0, _lib.F32, None) == _lib.ERR_NULL_POINTER
    assert lib.rglru_bwd(p, None, p, p, p, p, None, None, p, 1 << 20, None, None, None, None, None, 1, 2, 4, 8.0, _lib.F32, None) == _lib.ERR_NULL_POINTER
    assert lib.rglru_bwd(p, None, p, p, p, p, None, None, p, 1 << 20, None, None, None, p, p, 1, 2, 4, 8.0, _lib.F32, None) == _lib.ERR_NULL_POINTER
    assert lib.rglru_bwd(p, None, p, p, p, p, None, None, None, 0, None, None, None, None, p, 1, 2, 4, 8.0, _lib.F32, None) == _lib.ERR_WORKSPACE
    # shapes
    assert lib.rglru_fwd(p, p, p, p, None, None, p, None, None, 0, 0, 2, 4, 8.0, _lib.F32, None) == _lib.ERR_BAD_SHAPE
    assert lib.rglru_fwd(p, p, p, p, None, None, p, None, None, 0, 70000, 2, 4, 8.0, _lib.F32, None) == _lib.ERR_BAD_SHAPE
    assert lib.rglru_decode_step(p, p, p, p, p, None, p, 1, -1, 8.0, _lib.F32, None) == _lib.ERR_BAD_SHAPE
    # alignment (fp32 pointer off by two bytes)
    assert lib.rglru_fwd(p + 2, p, p, p, None, None, p, None, None, 0, 1, 2, 4, 8.0, _lib.F32, None) == _lib.ERR_MISALIGNED
    # workspace
    assert lib.rglru_fwd(p, p, p, p, None, None, p, None, p, 4, 1, 2, 4, 8.0, _lib.F32, None) == _lib.ERR_WORKSPACE
    assert lib.rglru_bwd(p, None, p, p, p, p, None, None, None, 0, p, p, p, p, None, 1, 2, 4, 8.0, _lib.F32, None) == _lib.ERR_WORKSPACE
    assert lib.rglru_conv_bwd(p, p, p, None, None, p, p, None, None, None, 0, 1, 2, 4, _lib.F32, None) == _lib.ERR_WORKSPACE
    assert lib.rglru_linear_scan_fwd(None, p, None, p, 1, 2, 4, None) == _lib.ERR_NULL_POINTER
    # grouped gate layout: x, u, gate_bias, branch, lambda, h0, tok, out, h_last, ws, ws_bytes, B, T, D, gate_width, ...
    big = (ctypes.c_float * 4096)()
    q = (ctypes.addressof(big) + 15) // 16 * 16
    assert lib.rglru_grouped_fwd(q, q, None, None, q, None, None, q, None, None, 0, 1, 2, 128, 48, 8.0, _lib.F32, None) == _lib.ERR_BAD_SHAPE
    assert lib.rglru_grouped_fwd(q, q, None, None, q, None, None, q, None, None, 0, 1, 2, 128, 64, 8.0, 5, None) == _lib.ERR_BAD_DTYPE
    assert lib.rglru_grouped_fwd(q, q + 4, None, None, q, None, None, q, None, None, 0, 1, 2, 128, 64, 8.0, _lib.F32, None) == _lib.ERR_MISALIGNED
    assert lib.rglru_grouped_fwd(q, None, None, None, q, None, None, q, None, None, 0, 1, 2, 128, 64, 8.0, _lib.F32, None) == _lib.ERR_NULL_POINTER
    assert lib.rglru_grouped_bwd(q, None, q, q, None, q, q, None, None, q, 1 << 20, q, q, None, q, None, None, 1, 2, 128, 64, 8.0, _lib.F32, None) == _lib.ERR_NULL_POINTER
    assert lib.rglru_grouped_bwd(q, None, q, q, None, None, q, None, None, q, 8, q, q, None, q, None, None, 1, 2, 128, 64, 8.0, _lib.F32, None) == _lib.ERR_WORKSPACE
    # column sums: size of the partial rows, and the argument checks (no launch: every call is refused)
    assert lib.rglru_column_sums_workspace_bytes(0, 8) == 0
    need = lib.rglru_column_sums_workspace_bytes(32768, 1024)
    assert need % (1024 * 4) == 0 and 0 < need <= 4 * 148 * 1024 * 4
    assert lib.rglru_column_sums_workspace_bytes(10, 8) == 8 * 4          # fewer than 64 rows: one row block
    assert lib.rglru_column_sums(q, q, q, 1 << 20, 4, 8, 5, None) == _lib.ERR_BAD_DTYPE
    assert lib.rglru_column_sums(None, q, q, 1 << 20, 4, 8, _lib.F32, None) == _lib.ERR_NULL_POINTER
    assert lib.rglru_column_sums(q, q, q, 1 << 20, 0, 8, _lib.F32, None) == _lib.ERR_BAD_SHAPE
    assert lib.rglru_column_sums(q, q, q, 4, 4, 8, _lib.F32, None) == _lib.ERR_WORKSPACE
    assert lib.rglru_column_sums(q + 2, q, q, 1 << 20, 4, 8, _lib.F32, None) == _lib.ERR_MISALIGNED
    # branch merge: x, conv_w, conv_b, conv_state, u_r, u_i, branch, lambda, h0, tok, out, h_last, ws, ws_bytes, ...
    assert lib.rglru_merge_fwd(p, None, None, None, p, p, None, p, None, None, p, None, None, 0, 1, 2, 4, 8.0, _lib.F32, None) == _lib.ERR_NULL_POINTER
    assert lib.rglru_merge_fwd(p, None, None, None, p, p, p, p, None, None, p, None, None, 0, 1, 2, 4, 8.0, 3, None) == _lib.ERR_BAD_DTYPE
    assert lib.rglru_merge_fwd(p, None, None, None, p, p, p + 2, p, None, None, p, None, None, 0, 1, 2, 4, 8.0, _lib.F32, None) == _lib.ERR_MISALIGNED
    assert lib.rglru_merge_bwd(p, None, p, None, None, None, p, p, p, p, None, None, p, 4, p, p, p, p, p, None, 1, 2, 4, 8.0, _lib.F32, None) == _lib.ERR_WORKSPACE
    assert lib.rglru_merge_bwd(p, None, p, None, None, None, p, p, p, p, None, None, p, 1 << 20, p, p, p, None, p, None, 1, 2, 4, 8.0, _lib.F32, None) == _lib.ERR_NULL_POINTER
    assert lib.rglru_conv_fwd(p, None, None, None, None, p, None, 1, 2, 4, _lib.F32, None) == _lib.ERR_NULL_POINTER


def test_status_codes_map_to_reference_exception_classes():
    from griffin_b200 import _lib
    with pytest.raises(ValueError):
        _lib.check(_lib.ERR_BAD_SHAPE, "x")
    with pytest.raises(TypeError):
        _lib.check(_lib.ERR_BAD_DTYPE, "x")
    with pytest.raises(RuntimeError, match="CUDA"):
        _lib.check(_lib.ERR_UNSUPPORTED, "x")
    _lib.check(_lib.OK, "x")


def test_module_rejects_what_the_reference_rejects():
    from griffin_b200 import RG_LRU, RecurrentBlock, linear_scan
    with pytest.raises(ValueError, match="Unknown RG-LRU scan mode"):
        RG_LRU(8, scan_mode="nonsense")
    with pytest.raises(ValueError, match="reference"):
        RG_LRU(8, scan_mode="sequential")
    m = RG_LRU(8, gate_blocks=4)
    assert m.scan_mode == "cuda" and RG_LRU(8, scan_mode="auto").scan_mode == "cuda"
    with pytest.raises(ValueError, match="expects \\[batch, sequence, width\\]"):
        m(torch.randn(2, 8))
    with pytest.raises(ValueError, match="Expected width"):
        m(torch.randn(2, 3, 9))
    with pytest.raises(ValueError, match="reset_mask"):
        m(torch.randn(2, 3, 8), reset_mask=torch.zeros(2, 4, dtype=torch.bool))
    with pytest.raises(ValueError, match="ht_minus_1"):
        m(torch.randn(2, 3, 8), torch.zeros(2, 7))
    # no CPU fallback: an explicit CUDA request on CPU tensors fails loudly (reference: tests/test_rglru.py:112-119)
    with pytest.raises(RuntimeError, match="CUDA"):
        m(torch.randn(2, 3, 8))
    with pytest.raises(RuntimeError, match="CUDA"):
        linear_scan(torch.rand(1, 2, 4), torch.rand(1, 2, 4), torch.zeros(1, 4))
    with pytest.raises(ValueError):
        RecurrentBlock(8, 8, conv_kernel_size=0)
    blk = RecurrentBlock(8, 12)
    with pytest.raises(ValueError, match="expects \\[batch, sequence, width\\]"):
        blk(torch.randn(3, 8))


def test_parameter_names_and_shapes_match_reference_checkpoints():
    """State dicts written by the reference load unchanged (names and shapes of griffin/griffin.py:138-141, 176, 379-389)."""
    from griffin_b200 import RG_LRU, RecurrentBlock
    case = load_golden("block_grads")
    blk = RecurrentBlock(16, 32, gate_blocks=4)
    blk.load_state_dict(params_of(case), strict=True)
    assert blk.temporal_conv.weight.shape == (32, 1, 4)
    assert blk.rg_lru.recurrence_gate.weight.shape == (4, 8, 8)
    m = RG_LRU(64, gate_blocks=16)
    assert m.recurrence_gate.weight.shape == (16, 4, 4) and m.Lambda.shape == (64,)
    a_pow_c = torch.sigmoid(m.Lambda.detach()) ** 8
    assert a_pow_c.min() >= 0.9 - 1e-4 and a_pow_c.max() <= 0.999 + 1e-4


def test_block_diagonal_linear_matches_oracle_einsum():
    from griffin_b200 import BlockDiagonalLinear
    from oracle import rglru_oracle as orc
    torch.manual_seed(0)
    lin = BlockDiagonalLinear(24, 4)
    with torch.no_grad():
        lin.bias.normal_()
    x = torch.randn(3, 5, 24)
    torch.testing.assert_close(lin(x), orc.block_diagonal_linear(x, lin.weight, lin.bias), atol=1e-6, rtol=1e-6)


def test_token_flags_and_positions():
    from griffin_b200 import _lib, token_flags
    from griffin_b200.modules import _last_real_position, _positions
    from oracle import rglru_oracle as orc
    assert token_flags(2, 3, "cpu") is None
    seg = torch.tensor([[0, 1, 2, 3, 4, 0, 1], [5, 6, 0, 1, 2, 3, 4]])
    active = torch.ones(2, 7, dtype=torch.bool)
    active[1, 5:] = False
    flags = token_flags(2, 7, "cpu", reset=seg == 0, active=active, segment_pos=seg, padded=~active.all())
    assert flags.dtype == torch.uint8
    assert flags[0].tolist() == [3 | 4 | 16, 2, 1, 0, 0, 3 | 4 | 16, 2]
    assert flags[1].tolist() == [0, 0, 3 | 4 | 16, 2, 1, _lib.TOK_INACTIVE, _lib.TOK_INACTIVE]
    x = torch.zeros(2, 7, 1)
    prev = torch.tensor([3, -1])
    got = _positions(x, None, prev, active)
    want = orc.resolve_positions(2, 7, None, prev, active)
    assert torch.equal(got, want)
    assert torch.equal(_positions(x, None, None, None), orc.resolve_positions(2, 7, None, None, None))
    assert torch.equal(_last_real_position(got, active, prev), orc.last_position(want, active, prev))
    none_active = torch.zeros(2, 7, dtype=torch.bool)
    assert torch.equal(_last_real_position(got, none_active, prev), orc.last_position(want, none_active, prev))


def test_missing_library_is_a_loud_error(monkeypatch, tmp_path):
    from griffin_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "absent.so"))
    with pytest.raises(RuntimeError, match="no CPU or Triton fallback"):
        _lib.load()


def test_scan_self_check_says_no_without_a_cuda_device():
    """tests/test_rglru.py:122-124 of the reference: the usability probe is False for the CPU."""
    from griffin_b200 import cuda_scan_is_usable
    assert cuda_scan_is_usable("cpu") is False
    with pytest.raises(RuntimeError):
        cuda_scan_is_usable("cpu", strict=True)


def test_stable_partition_matches_a_stable_sort():
    """Rows whose padding is not right padding are reordered real-tokens-first; the indices come from running counts
    and must equal those of a stable sort of the mask (behaviour pinned by the reference: padding neither enters the
    conv history nor moves the state, griffin/griffin.py:488-510)."""
    from griffin_b200.modules import _stable_partition
    gen = torch.Generator().manual_seed(11)
    for steps in (1, 2, 7, 64, 129):
        mask = torch.rand(6, steps, generator=gen) < 0.6
        mask[0] = True
        mask[1] = False
        order, restore = _stable_partition(mask)
        want_order = torch.argsort((~mask).to(torch.uint8), dim=1, stable=True)
        assert torch.equal(order, want_order)
        assert torch.equal(restore, torch.argsort(want_order, dim=1))
        assert torch.equal(torch.gather(order, 1, restore), torch.arange(steps).expand(6, steps))


def test_row_permutation_has_a_gather_backward_and_the_padding_kind_is_remembered_per_mask_object():
    from griffin_b200.modules import _flat_rows, _needs_partition, _PermuteRows, _stable_partition
    gen = torch.Generator().manual_seed(12)
    mask = torch.rand(3, 9, generator=gen) < 0.6
    order, restore = _stable_partition(mask)
    x = torch.randn(3, 9, 4, dtype=torch.float64, generator=gen).requires_grad_(True)
    flat_order, flat_restore = _flat_rows(order), _flat_rows(restore)
    moved = _PermuteRows.apply(x, flat_order, flat_restore)
    plain = x.gather(1, order[..., None].expand(-1, -1, 4))
    assert torch.equal(moved, plain)
    g = torch.randn(3, 9, 4, dtype=torch.float64, generator=gen)
    assert torch.equal(torch.autograd.grad(moved, x, g)[0], torch.autograd.grad(plain, x, g)[0])
    assert torch.equal(_PermuteRows.apply(moved, flat_restore, flat_order), x)
    right = torch.ones(2, 5, dtype=torch.bool)
    right[:, 3:] = False
    assert _needs_partition(right, right) is False and _needs_partition(right, right) is False
    right[0, 4] = True                     # an in-place change is a new version: the answer is worked out again
    assert _needs_partition(right, right) is True
    assert _needs_partition(right.clone(), right.clone()) is True      # another object: no stale hit


def test_mask_plans_are_shared_per_tensor_object_and_version():
    from griffin_b200.modules import _shared_between_blocks
    calls = []

    def build():
        calls.append(1)
        return len(calls)

    pos, mask = torch.arange(6).reshape(1, 6), torch.ones(1, 6, dtype=torch.bool)
    cpu = torch.device("cpu")
    assert _shared_between_blocks((pos, mask), cpu, build) == 1
    assert _shared_between_blocks((pos, mask), cpu, build) == 1            # same objects, same versions: remembered
    assert _shared_between_blocks((pos, None), cpu, build) == 2            # another combination
    mask[0, 5] = False                                                     # in-place change: a new version
    assert _shared_between_blocks((pos, mask), cpu, build) == 3
    assert _shared_between_blocks((pos.clone(), mask), cpu, build) == 4    # another object with equal content
    with torch.inference_mode():
        assert _shared_between_blocks((pos, mask), cpu, build) == 5        # nothing is remembered here ...
    assert _shared_between_blocks((pos, mask), cpu, build) == 3            # ... and the earlier entry is untouched
    assert _shared_between_blocks((None, None), cpu, build) == 6           # no owner: nothing to key on


def test_memos_leave_inference_tensors_alone():
    from griffin_b200.modules import _needs_partition, _shared_between_blocks
    with torch.inference_mode():
        mask = torch.ones(2, 5, dtype=torch.bool)
        mask[0, :2] = False
    calls = []
    for _ in range(2):       # an inference tensor tracks no version: worked out every time, never an error
        assert _needs_partition(mask, mask) is True
        assert _shared_between_blocks((None, mask), torch.device("cpu"), lambda: calls.append(1) or len(calls)) == len(calls)
    assert len(calls) == 2
