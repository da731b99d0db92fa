"""Tensor layouts of the W4A4 path (oracle; test infrastructure, never shipped).

Two families:

``ref_*``    the reference's packed layouts: register-fragment order of its
             ``mma.sync`` kernels.  Weight-side ones are produced by
             ``NunchakuWeightPacker`` (nunchaku/lora/flux/packer.py:187-398);
             activation-side ones are written by the reference kernels
             (src/kernels/zgemm/gemm_w4a4.cuh:85-187,429-523,930-1043,
             gemm_base.cuh:97-154,452-468, lora.cuh:43-61).
``native_*`` the layouts the sm_100a kernels of this repository consume
             (row-major K-major codes for TMA, 512-byte scale-factor atoms for
             ``tcgen05.cp``, plain row-major fp32 low-rank activations).

Every layout is expressed as a permutation ``perm`` of logical flat indices
(memory position i holds logical element perm[i]) so that pack and unpack are
one gather / one scatter and provably inverse of each other.
"""
from __future__ import annotations

import functools

import torch


def _idx(*shape: int) -> torch.Tensor:
    n = 1
    for s in shape:
        n *= s
    return torch.arange(n, dtype=torch.int64).reshape(*shape)


def _gather(logical: torch.Tensor, perm: torch.Tensor) -> torch.Tensor:
    return logical.reshape(-1)[perm]


def _scatter(packed: torch.Tensor, perm: torch.Tensor) -> torch.Tensor:
    out = torch.empty_like(packed.reshape(-1))
    out[perm] = packed.reshape(-1)
    return out


# ---------------------------------------------------------------------------
# nibble <-> byte helpers (lowest nibble = lowest k, gemm_w4a4.cuh:163-187)
# ---------------------------------------------------------------------------
def nibbles_to_bytes(nib: torch.Tensor) -> torch.Tensor:
    nib = nib.reshape(-1, 2).to(torch.uint8)
    return (nib[:, 0] & 0xF) | ((nib[:, 1] & 0xF) << 4)


def bytes_to_nibbles(b: torch.Tensor) -> torch.Tensor:
    b = b.reshape(-1).view(torch.uint8) if b.dtype in (torch.int8, torch.uint8) else b.reshape(-1)
    b = b.to(torch.uint8)
    return torch.stack([b & 0xF, b >> 4], dim=1).reshape(-1)


# ---------------------------------------------------------------------------
# reference layouts
# ---------------------------------------------------------------------------
@functools.lru_cache(maxsize=64)
def _perm_ref_act_codes(M: int, K: int) -> torch.Tensor:
    # memory: [M/256][K/64][warp 8][mtile 2][g 8][t 4][kh 2][half 2][j 8] nibbles
    # logical row = bm*256 + w*32 + mt*16 + half*8 + g ; k = bk*64 + kh*32 + t*8 + j
    assert M % 256 == 0 and K % 64 == 0
    i = _idx(M // 256, 8, 2, 2, 8, K // 64, 2, 4, 8)  # bm w mt half g bk kh t j
    return i.permute(0, 5, 1, 2, 4, 7, 6, 3, 8).reshape(-1)


@functools.lru_cache(maxsize=64)
def _perm_ref_wgt_codes(N: int, K: int) -> torch.Tensor:
    # memory: [N/128][K/64][ntile 8][g 8][t 4][half 2][kh 2][j 8] nibbles
    assert N % 128 == 0 and K % 64 == 0
    i = _idx(N // 128, 8, 2, 8, K // 64, 2, 4, 8)  # bn nt half g bk kh t j
    return i.permute(0, 4, 1, 3, 6, 2, 5, 7).reshape(-1)


def ref_pack_act_codes(codes: torch.Tensor) -> torch.Tensor:
    """[M_pad, K] nibble values -> uint8 [M_pad, K/2] in reference fragment order."""
    M, K = codes.shape
    return nibbles_to_bytes(_gather(codes, _perm_ref_act_codes(M, K))).reshape(M, K // 2)


def ref_unpack_act_codes(packed: torch.Tensor, K: int) -> torch.Tensor:
    M = packed.shape[0]
    return _scatter(bytes_to_nibbles(packed), _perm_ref_act_codes(M, K)).reshape(M, K)


def ref_pack_wgt_codes(codes: torch.Tensor) -> torch.Tensor:
    """[N, K] nibble values -> int8 [N, K/2] (== NunchakuWeightPacker.pack_weight)."""
    N, K = codes.shape
    return nibbles_to_bytes(_gather(codes, _perm_ref_wgt_codes(N, K))).reshape(N, K // 2).view(torch.int8)


def ref_unpack_wgt_codes(packed: torch.Tensor, K: int) -> torch.Tensor:
    N = packed.shape[0]
    return _scatter(bytes_to_nibbles(packed), _perm_ref_wgt_codes(N, K)).reshape(N, K)


@functools.lru_cache(maxsize=64)
def _perm_ref_ascales(M: int, G: int) -> torch.Tensor:
    # INT4 activation scales, logical [G = K/64, M]; memory
    # [M/256][G][warp 8][q 2][g 8][e 2]; row = bm*256 + w*32 + q*16 + e*8 + g
    i = _idx(G, M // 256, 8, 2, 2, 8)  # kg bm w q e g
    return i.permute(1, 0, 2, 3, 5, 4).reshape(-1)


def ref_pack_ascales(s: torch.Tensor) -> torch.Tensor:
    """logical [K/64, M_pad] -> same shape, reference memory order (gemm_base.cuh:452-468)."""
    G, M = s.shape
    return _gather(s, _perm_ref_ascales(M, G)).reshape(G, M)


def ref_unpack_ascales(p: torch.Tensor) -> torch.Tensor:
    G, M = p.shape
    return _scatter(p, _perm_ref_ascales(M, G)).reshape(G, M)


@functools.lru_cache(maxsize=64)
def _perm_ref_vec128(N: int, G: int) -> torch.Tensor:
    # INT4 weight scales / bias / smooth / wcscales, logical [G, N]; memory
    # [N/128][G][a 8][c 4][b 2][d 2]; n = bn*128 + a*16 + b*8 + c*2 + d
    # (gemm_base.cuh:97-126, packer.py:241-301)
    i = _idx(G, N // 128, 8, 2, 4, 2)  # kg bn a b c d
    return i.permute(1, 0, 2, 4, 3, 5).reshape(-1)


def ref_pack_wscales(s: torch.Tensor) -> torch.Tensor:
    """logical [K/64, N] -> reference order (== pack_scale(scale[N, K/64], 64))."""
    G, N = s.shape
    return _gather(s, _perm_ref_vec128(N, G)).reshape(G, N)


def ref_unpack_wscales(p: torch.Tensor) -> torch.Tensor:
    G, N = p.shape
    return _scatter(p, _perm_ref_vec128(N, G)).reshape(G, N)


def ref_pack_vector(v: torch.Tensor) -> torch.Tensor:
    """bias / smooth_factor / wcscales [N] -> reference order (pack_scale(..., -1))."""
    return _gather(v, _perm_ref_vec128(v.numel(), 1))


def ref_unpack_vector(p: torch.Tensor) -> torch.Tensor:
    return _scatter(p, _perm_ref_vec128(p.numel(), 1))


@functools.lru_cache(maxsize=64)
def _perm_ref_amscales(M: int, G16: int) -> torch.Tensor:
    # NVFP4 activation micro-scales, logical [G16 = K/16, M] bytes; memory
    # [M/256][K/64][warp 8][lane 32][kg 4]; row in warp = ((l%4)/2)*16 + (l%2)*8 + l/4
    # (gemm_w4a4.cuh:144-155)
    i = _idx(G16 // 4, 4, M // 256, 8, 2, 2, 8)  # bk kg bm w tile e q   (row = tile*16 + e*8 + q)
    # lane = q*4 + tile*2 + e
    return i.permute(2, 0, 3, 6, 4, 5, 1).reshape(-1)


def ref_pack_amscales(s: torch.Tensor) -> torch.Tensor:
    G16, M = s.shape
    return _gather(s, _perm_ref_amscales(M, G16)).reshape(G16, M)


def ref_unpack_amscales(p: torch.Tensor) -> torch.Tensor:
    G16, M = p.shape
    return _scatter(p, _perm_ref_amscales(M, G16)).reshape(G16, M)


@functools.lru_cache(maxsize=64)
def _perm_ref_wmscales(N: int, G16: int) -> torch.Tensor:
    # NVFP4 weight micro-scales, logical [G16, N] bytes; memory
    # [N/128][K/64][d 8][c 4][s 4][kg 4]; n = bn*128 + s*32 + c*8 + d (packer.py:303-360)
    i = _idx(G16 // 4, 4, N // 128, 4, 4, 8)  # bk kg bn s c d
    return i.permute(2, 0, 5, 4, 3, 1).reshape(-1)


def ref_pack_wmscales(s: torch.Tensor) -> torch.Tensor:
    """logical [K/16, N] e4m3 bytes -> reference order (== pack_micro_scale(scale[N, K/16]))."""
    G16, N = s.shape
    return _gather(s, _perm_ref_wmscales(N, G16)).reshape(G16, N)


def ref_unpack_wmscales(p: torch.Tensor) -> torch.Tensor:
    G16, N = p.shape
    return _scatter(p, _perm_ref_wmscales(N, G16)).reshape(G16, N)


@functools.lru_cache(maxsize=64)
def _perm_ref_lora_wgt(C: int, R: int, down: bool) -> torch.Tensor:
    # memory [C/16][R/16][g 8][t 4][nh 2][kh 2][e 2] (packer.py:362-398, lora.cuh:43-44)
    #  up   (logical [N=C, R]): n = cp*16 + nh*8 + g ; r = rp*16 + kh*8 + t*2 + e
    #  down (logical [R, K=C]): r = rp*16 + nh*8 + g ; c = cp*16 + kh*8 + t*2 + e
    if down:
        i = _idx(R // 16, 2, 8, C // 16, 2, 4, 2)  # rp nh g cp kh t e
        return i.permute(3, 0, 2, 5, 1, 4, 6).reshape(-1)
    i = _idx(C // 16, 2, 8, R // 16, 2, 4, 2)  # cp nh g rp kh t e
    return i.permute(0, 3, 2, 5, 1, 4, 6).reshape(-1)


def ref_pack_lora_up(w: torch.Tensor) -> torch.Tensor:
    """logical [N, R] -> packed, nominal shape [N, R]."""
    N, R = w.shape
    return _gather(w, _perm_ref_lora_wgt(N, R, False)).reshape(N, R)


def ref_unpack_lora_up(p: torch.Tensor) -> torch.Tensor:
    N, R = p.shape
    return _scatter(p, _perm_ref_lora_wgt(N, R, False)).reshape(N, R)


def ref_pack_lora_down(w: torch.Tensor) -> torch.Tensor:
    """logical [R, K] -> packed, nominal shape [K, R] (the module's ``proj_down``)."""
    R, K = w.shape
    return _gather(w, _perm_ref_lora_wgt(K, R, True)).reshape(K, R)


def ref_unpack_lora_down(p: torch.Tensor) -> torch.Tensor:
    """packed [K, R] -> logical [R, K]."""
    K, R = p.shape
    return _scatter(p, _perm_ref_lora_wgt(K, R, True)).reshape(R, K)


@functools.lru_cache(maxsize=64)
def _perm_ref_lora_act(M: int, R: int) -> torch.Tensor:
    # logical [M, R] fp32; memory [M/256][R/16][warp 8][mtile 2][rh 2][half 2][e 2][g 8][t 4]
    # row = bm*256 + w*32 + mt*16 + half*8 + g ; rank = rt*16 + rh*8 + 2t + e (lora.cuh:61-94)
    i = _idx(M // 256, 8, 2, 2, 8, R // 16, 2, 4, 2)  # bm w mt half g rt rh t e
    return i.permute(0, 5, 1, 2, 6, 3, 8, 4, 7).reshape(-1)


def ref_pack_lora_act(a: torch.Tensor) -> torch.Tensor:
    M, R = a.shape
    return _gather(a, _perm_ref_lora_act(M, R)).reshape(M, R)


def ref_unpack_lora_act(p: torch.Tensor) -> torch.Tensor:
    M, R = p.shape
    return _scatter(p, _perm_ref_lora_act(M, R)).reshape(M, R)


# ---------------------------------------------------------------------------
# native (sm_100a) layouts
# ---------------------------------------------------------------------------
def native_pack_codes(codes: torch.Tensor) -> torch.Tensor:
    """[rows, K] nibble values -> uint8 [rows, K/2], row-major, low nibble = even k."""
    rows, K = codes.shape
    return nibbles_to_bytes(codes).reshape(rows, K // 2)


def native_unpack_codes(packed: torch.Tensor, K: int) -> torch.Tensor:
    return bytes_to_nibbles(packed).reshape(packed.shape[0], K)


@functools.lru_cache(maxsize=64)
def _perm_native_sf(rows: int, G16: int) -> torch.Tensor:
    # logical [G16 = K/16, rows] bytes; memory [rows/128][K/64][r0 32][r1 4][kg 4]
    # (row = blk*128 + r1*32 + r0): one 512-byte atom per (128 rows, 64 k), the
    # image tcgen05.cp.32x128b.warpx4 moves into 4 TMEM columns.
    i = _idx(G16 // 4, 4, rows // 128, 4, 32)  # bk kg blk r1 r0
    return i.permute(2, 0, 4, 3, 1).reshape(-1)


def native_pack_sf(s: torch.Tensor) -> torch.Tensor:
    G16, rows = s.shape
    return _gather(s, _perm_native_sf(rows, G16)).reshape(G16, rows)


def native_unpack_sf(p: torch.Tensor) -> torch.Tensor:
    G16, rows = p.shape
    return _scatter(p, _perm_native_sf(rows, G16)).reshape(G16, rows)
