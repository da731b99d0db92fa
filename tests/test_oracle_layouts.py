"""oracle.layouts against the reference packer's own outputs (tests/golden/packer_golden.npz)
and pack/unpack round trips of the activation-side layouts."""
import numpy as np
import torch

from oracle import layouts as L


def _bf16(a):
    return torch.from_numpy(np.ascontiguousarray(a)).view(torch.bfloat16)


def test_weight_codes_match_reference_packer(golden):
    codes = torch.from_numpy(golden["wgt_codes_in"]).to(torch.int32) & 0xF
    packed = L.ref_pack_wgt_codes(codes.to(torch.uint8))
    assert np.array_equal(packed.view(torch.uint8).numpy(), golden["wgt_codes_packed"])
    assert torch.equal(L.ref_unpack_wgt_codes(packed, codes.shape[1]).to(torch.int32), codes)


def test_int4_wscales_match_reference_packer(golden):
    ws = _bf16(golden["wscales_in"])  # [N, K/64]
    packed = L.ref_pack_wscales(ws.t().contiguous())  # logical [K/64, N]
    assert np.array_equal(packed.view(torch.int16).numpy(), golden["wscales_packed"])
    assert torch.equal(L.ref_unpack_wscales(packed), ws.t())


def test_vector_matches_reference_packer(golden):
    v = _bf16(golden["vector_in"])
    packed = L.ref_pack_vector(v)
    assert np.array_equal(packed.view(torch.int16).numpy(), golden["vector_packed"])
    assert torch.equal(L.ref_unpack_vector(packed), v)
    # the lane map documented at gemm_base.cuh:100-112: lane 0 holds 0,1,8,9 ; lane 31 holds 118,119,126,127
    idx = golden["vector_index_packed"]
    assert idx[:4].tolist() == [0, 1, 8, 9] and idx[-4:].tolist() == [118, 119, 126, 127]
    mine = L.ref_pack_vector(torch.arange(128, dtype=torch.int16))
    assert mine.tolist() == idx.tolist()


def test_nvfp4_wmscales_match_reference_packer(golden):
    ms = torch.from_numpy(golden["wmscales_in"])  # [N, K/16] bytes
    packed = L.ref_pack_wmscales(ms.t().contiguous())
    assert np.array_equal(packed.numpy(), golden["wmscales_packed"])
    assert torch.equal(L.ref_unpack_wmscales(packed), ms.t())


def test_lora_weights_match_reference_packer(golden):
    up = _bf16(golden["lora_up_in"])
    pu = L.ref_pack_lora_up(up)
    assert np.array_equal(pu.view(torch.int16).numpy(), golden["lora_up_packed"])
    assert torch.equal(L.ref_unpack_lora_up(pu), up)
    down = _bf16(golden["lora_down_in"])  # [R, K]
    pd = L.ref_pack_lora_down(down)
    assert np.array_equal(pd.view(torch.int16).numpy(), golden["lora_down_packed"])
    assert torch.equal(L.ref_unpack_lora_down(pd), down)


def test_activation_layout_round_trips():
    g = torch.Generator().manual_seed(0)
    M, K, R = 512, 256, 32
    codes = torch.randint(0, 16, (M, K), generator=g, dtype=torch.uint8)
    assert torch.equal(L.ref_unpack_act_codes(L.ref_pack_act_codes(codes), K), codes)
    assert torch.equal(L.native_unpack_codes(L.native_pack_codes(codes), K), codes)
    s = torch.randint(0, 255, (K // 16, M), generator=g, dtype=torch.uint8)
    assert torch.equal(L.ref_unpack_amscales(L.ref_pack_amscales(s)), s)
    assert torch.equal(L.native_unpack_sf(L.native_pack_sf(s)), s)
    a = torch.randn(K // 64, M, generator=g).to(torch.bfloat16)
    assert torch.equal(L.ref_unpack_ascales(L.ref_pack_ascales(a)), a)
    la = torch.randn(M, R, generator=g)
    assert torch.equal(L.ref_unpack_lora_act(L.ref_pack_lora_act(la)), la)


def test_activation_code_lane_map():
    """Known-answer for the act fragment order (gemm_w4a4.cuh:163-187): lane l = 4g+t of
    warp 0 / m-tile 0 holds {x: (row g, k 8t..), y: (row g+8, k 8t..), z: (row g, k 32+8t..),
    w: (row g+8, k 32+8t..)}."""
    M, K = 256, 64
    rows = torch.arange(M).view(M, 1).expand(M, K)
    ks = torch.arange(K).view(1, K).expand(M, K)
    # encode row in one plane and k in another and check the first uint4 of lane 5 (g=1, t=1)
    pr = L._gather(rows.contiguous(), L._perm_ref_act_codes(M, K)).view(-1, 4, 8)
    pk = L._gather(ks.contiguous(), L._perm_ref_act_codes(M, K)).view(-1, 4, 8)
    lane = 5
    assert pr[lane, :, 0].tolist() == [1, 9, 1, 9]
    assert pk[lane, :, 0].tolist() == [8, 8, 40, 40]
    assert pk[lane, 0].tolist() == list(range(8, 16))


def test_amscale_lane_map():
    """gemm_w4a4.cuh:144-155: lane i holds row i/4 + 8*(i%2) of m-tile (i%4)/2."""
    M, G16 = 256, 4
    rows = torch.arange(M).view(1, M).expand(G16, M).contiguous()
    pr = L._gather(rows, L._perm_ref_amscales(M, G16)).view(-1, 4)
    for lane in range(32):
        assert pr[lane, 0].item() == ((lane % 4) // 2) * 16 + lane // 4 + 8 * (lane % 2)
