"""CPU-side checks of the C-ABI library: it loads, exports every symbol the public header declares, refuses bad
arguments with the documented codes, and its HOST-ONLY producers are bit-exact against the reference goldens and the
oracle.  No compute entry is called here (no GPU)."""
import ctypes as C
import os
import re

import numpy as np
import pytest
import torch

import quactlize_b200 as qb
from conftest import ROOT, load_golden
from oracle import kquant as kq
from quactlize_b200 import _lib, synth


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "quactlize_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(quactlize_(?:ppu|b200)_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = _declared_symbols()
    assert len(names) > 30
    h = C.CDLL(_lib.LIB_PATH)
    missing = [n for n in names if not hasattr(h, n)]
    assert not missing, missing


def test_binding_table_matches_header():
    assert sorted(_lib.SIGNATURES) == _declared_symbols()
    _lib.lib()


def test_reference_loader_mandatory_symbols_present():
    # quactlize/csrc/preprocess/thop/ppu_backend.cpp:85-108 refuses a library that lacks any of these
    h = C.CDLL(_lib.LIB_PATH)
    for n in ("quactlize_ppu_vecdot", "quactlize_ppu_vecdot_moe", "quactlize_ppu_dequantize", "quactlize_ppu_prepass",
              "quactlize_ppu_gemv_lowbit"):
        assert hasattr(h, n)


def test_argument_refusals_need_no_device():
    L = _lib.lib()
    assert L.quactlize_ppu_vecdot(None, 144, None, None, 4, 1, 99) == 1           # unknown qtype
    assert L.quactlize_ppu_vecdot(None, 143, None, None, 4, 1, 12) == 10          # wrong block size
    assert L.quactlize_ppu_vecdot_dense(None, 144, None, None, 4, 1, 99) == 3
    assert L.quactlize_ppu_vecdot_dense(None, 144, None, None, 0, 1, 12) == 12
    assert L.quactlize_ppu_vecdot_moe(None, 144, None, None, None, 8, 1, 2, 4, 2, 99) == 2
    assert L.quactlize_ppu_vecdot_moe(None, 144, None, None, None, 0, 1, 2, 4, 2, 12) == 11
    assert L.quactlize_ppu_dequantize(None, 144, None, 0, 12) == 12
    assert L.quactlize_ppu_prepass(None, 12, None, None, 4, None, None, 8, 12, 3) == 4
    assert L.quactlize_ppu_prepass_unit(None, None, None, 256, 256, 1, 12, 0) == 7
    assert L.quactlize_ppu_gemv_lowbit(None, None, None, None, None, None, 1, 256, 256, 32, 99, 0, None, 1) == 6
    assert L.quactlize_ppu_bc_gemv(None, None, None, None, None, None, 1, 256, 256, 0, 1, 12) == 13
    assert L.quactlize_ppu_units_bytes(256, 256, 99) == -1
    assert L.quactlize_ppu_units_bytes(100, 256, 12) == -1
    assert L.quactlize_ppu_units_bytes(256, 256, 14) == -1                        # Q6_K pairs two superblocks
    assert L.quactlize_ppu_units_bytes(256, 512, 14) == 256 * 36
    assert L.quactlize_ppu_units_bytes(256, 512, 12) == 256 * 2 * 16
    assert L.quactlize_ppu_gemv_lowbit_config_valid_v1(1, 4096, 4096, 32, 12, None) == 1
    assert L.quactlize_ppu_gemv_lowbit_config_valid_v1(1, 4096, 4096, 16, 12, None) == 0
    assert L.quactlize_ppu_gemv_lowbit_config_valid_v1(1, 4096, 4096, 32, 12, b"64x64:32x32:s3") == 0
    assert L.quactlize_ppu_vecdot_moe_config_valid_v1(4, 256, 512, 32, 2, 3, 12, b"vecdot_moe") == 1
    cfg = (_lib.ConfigV2 * 2)()
    assert L.quactlize_ppu_list_valid_vecdot_moe_configs_v2(cfg, 2, 4, 256, 512, 32, 2, 3, 12) == 1
    assert cfg[0].enable_cuda_kernel and cfg[0].name == b"vecdot_moe"


def test_tensor_tactic_inventory():
    """Two tensor-core tactics are compiled; both are listed as valid for every valid shape and recognised by name."""
    L = _lib.lib()
    cfg = (_lib.ConfigV2 * 4)()
    assert L.quactlize_ppu_list_valid_dense_lowbit_configs_v2(cfg, 4, 64, 4096, 4096, 32, 12) == 2
    names = [cfg[i].name for i in range(2)]
    assert names == [b"256x256x64:tcgen05", b"128x128x64:tcgen05"]
    assert (cfg[0].tile_m, cfg[0].tile_n, cfg[1].tile_m, cfg[1].tile_n) == (256, 256, 128, 128)
    assert L.quactlize_ppu_list_valid_dense_lowbit_configs_v2(cfg, 4, 64, 4000, 4096, 32, 12) == 0       # n not a tile multiple
    for name in names:
        assert L.quactlize_ppu_dense_lowbit_config_valid_v1(64, 4096, 4096, 32, 12, name) == 1
        assert L.quactlize_ppu_grouped_fully_quantized_config_valid_v1(64, 4096, 4096, 32, 8, 64, 12, name) == 1
    assert L.quactlize_ppu_dense_lowbit_config_valid_v1(64, 4096, 4096, 32, 12, b"64x64x64:other") == 0
    assert L.quactlize_ppu_list_configs(None) == 3 and L.quactlize_ppu_list_grouped_configs(None) == 4
    # the split-K decode tactic belongs to the grouped routes only
    sk = b"128x128x64:tcgen05:splitk"
    assert L.quactlize_ppu_grouped_fully_quantized_config_valid_v1(64, 4096, 4096, 32, 8, 64, 12, sk) == 1
    assert L.quactlize_ppu_grouped_lowbit_config_valid_v1(64, 4096, 4096, 32, 8, 64, 12, sk) == 1
    assert L.quactlize_ppu_dense_lowbit_config_valid_v1(64, 4096, 4096, 32, 12, sk) == 0
    assert L.quactlize_ppu_list_valid_grouped_fully_quantized_configs_v2(cfg, 4, 64, 4096, 4096, 32, 8, 64, 12) == 3 and cfg[2].name == sk
    # its fp32 partial planes: the generic query, and the extra room the reference-shaped queries add for decode sizes
    assert L.quactlize_b200_gemm_plane_splitk_workspace_bytes_v1(512, 1536, 4) == 4 * 512 * 1536 * 4
    assert L.quactlize_b200_gemm_plane_splitk_workspace_bytes_v1(512, 1536, 0) == 8 * 512 * 1536 * 4
    assert L.quactlize_b200_gemm_plane_splitk_workspace_bytes_v1(512, 1536, 65) == -1
    assert L.quactlize_ppu_grouped_lowbit_workspace_bytes_v1(8, 1536, 2048, 32, 128, 12) == 256 + 8 * 128 * 8 * 1536 * 4 + 16
    assert L.quactlize_ppu_grouped_lowbit_workspace_bytes_v1(4096, 14336, 4096, 32, 8, 12) == 256      # prefill sizes: no split-K


def _eq(a, b):
    a = a.numpy() if isinstance(a, torch.Tensor) else np.asarray(a)
    b = np.asarray(b)
    assert a.shape == b.shape, (a.shape, b.shape)
    if a.dtype == np.float16:
        a, b = a.view(np.uint16), b.view(np.uint16)
    assert np.array_equal(a, b)


def test_prepare_gemv_host_producer_bit_exact(qtype):
    g = load_golden(qtype)
    low, high, scale, zero = qb.gguf_prepare_gemv(torch.from_numpy(g["blocks"]), int(g["n"]), int(g["k"]), qtype)
    _eq(low, g["low"]); _eq(high, g["high"]); _eq(scale, g["scale"]); _eq(zero, g["zero"])


def test_pack_units_host_producer_bit_exact(qtype):
    g = load_golden(qtype)
    units = qb.gguf_pack_units(torch.from_numpy(g["blocks"]), int(g["n"]), int(g["k"]), qtype)
    _eq(units[0], g["units"])


@pytest.mark.parametrize("experts", [1, 3])
def test_fully_quantized_round_trip(qtype, experts):
    n, k = 256, 512
    blocks = synth.kquant_blocks(qtype, experts * n * k // 256, seed=31 + qtype)
    tb = torch.from_numpy(blocks)
    if experts == 1:
        low, high, units = qb.gguf_prepare_fully_quantized_dense(tb, n, k, qtype)
        units4 = units.unsqueeze(0)
    else:
        low, high, units = qb.gguf_prepare_fully_quantized_grouped(tb, n, k, qtype, experts)
        units4 = units
    olow, ohigh, ounits = kq.prepare_fully_quantized(blocks, n, k, qtype, experts)
    _eq(low, olow); _eq(high, ohigh); _eq(units4, ounits)
    # byte-neutral: the artifact holds exactly the checkpoint's bytes
    assert low.numel() + high.numel() + units.numel() == blocks.size
    back = qb.gguf_recover_fully_quantized(low, high, units4, n, k, qtype)
    _eq(back, blocks)


def test_units_need_paired_superblocks():
    blocks = torch.from_numpy(synth.kquant_blocks(14, 256, seed=1))
    with pytest.raises(RuntimeError):
        qb.gguf_prepare_fully_quantized_dense(blocks, 256, 256, 14)


def test_shape_contract_errors():
    blocks = torch.from_numpy(synth.kquant_blocks(12, 16, seed=1))
    with pytest.raises(RuntimeError):
        qb.gguf_prepare_gemv(blocks, 8, 300, 12)
    with pytest.raises(RuntimeError):
        qb.gguf_prepare_gemv(blocks[:, :100].contiguous(), 8, 512, 12)
    with pytest.raises(RuntimeError):
        qb.gguf_dequantize(blocks, 9)


def test_header_is_c_and_a_c_caller_can_load_the_library(tmp_path):
    """The boundary is a C ABI: a C program that includes the header, dlopens the library and calls host-only entries."""
    import shutil
    import subprocess
    if shutil.which("gcc") is None:
        pytest.skip("no C compiler")
    here = os.path.dirname(os.path.abspath(__file__))
    exe = tmp_path / "c_abi_probe"
    subprocess.run(["gcc", "-std=c11", "-Wall", "-Werror", "-I", os.path.join(os.path.dirname(here), "include"),
                    os.path.join(here, "c_abi_probe.c"), "-o", str(exe), "-ldl"], check=True)
    r = subprocess.run([str(exe), _lib.LIB_PATH], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.startswith("ok 8192 ")


def test_pack_unit_reference_form_matches_golden(qtype):
    """The reference-form op (scale blocks + fp16 headers in, units out): the 3-D artifact form reproduces the units the
    reference's own op produced, and the 2-D row-wise form equals the artifact form of a single column."""
    import torch
    import quactlize_b200 as qb
    from quactlize_b200.formats import kquant_geometry
    g = load_golden(qtype)
    geo = kquant_geometry(qtype)
    n, k = int(g["n"]), int(g["k"])
    nsb = k // 256
    d_off, m_off, s_off = {10: (80, 82, 0), 11: (108, -1, 96), 12: (0, 2, 4), 13: (0, 2, 4), 14: (208, -1, 192)}[qtype]
    tb = torch.from_numpy(g["blocks"])
    sblk = tb[:, s_off:s_off + geo.scale_bytes].contiguous().view(n, nsb, geo.scale_bytes)
    d = tb[:, d_off:d_off + 2].contiguous().view(torch.float16).view(n, nsb)
    dm = tb[:, m_off:m_off + 2].contiguous().view(torch.float16).view(n, nsb) if m_off >= 0 else torch.empty(0, dtype=torch.float16)
    units = qb.gguf_pack_unit(sblk, d, dm, qtype)
    assert np.array_equal(units.numpy(), g["units"])
    col = 5
    rowwise = qb.gguf_pack_unit(sblk[col].contiguous(), d[col].contiguous(), dm[col].contiguous() if m_off >= 0 else dm, qtype)
    assert np.array_equal(rowwise.numpy(), g["units"][:, col, :])
    assert qb.gguf_scale_block_shape(qtype)[:4] == [geo.scale_bytes, geo.groups, geo.group_size, int(geo.has_min)]
    if geo.has_min:
        with pytest.raises(RuntimeError):
            qb.gguf_pack_unit(sblk, d, None, qtype)


def test_variant_builds_need_a_name_and_a_macro_the_sources_mention():
    """The ablation builds (`python -m quactlize_b200.build --variant NAME --define MACRO`) refuse what cannot work before
    any compiler runs: a name that is no identifier, no macro, a macro no source mentions."""
    from quactlize_b200 import build as qbuild
    for name, defines in (("no-dash", ["QB_SWAP_NOST"]), ("ok", []), ("ok", ["QB_NO_SUCH_SWITCH"])):
        with pytest.raises(ValueError):
            qbuild.build_variant(name, defines)
