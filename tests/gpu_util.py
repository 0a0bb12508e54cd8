"""Shared helpers of the GPU parity tests: seeded inputs, device round trips through the C ABI."""
import numpy as np

import ascb200 as ab
import oracle as orc

_inited = False


def dev():
    global _inited
    if not _inited:
        ab.init(0)
        _inited = True
    return ab


def f16_bits(a):
    return np.ascontiguousarray(a.astype(np.float16)).view(np.uint16)


def bf16_bits(a):
    """float32 -> bf16 bit patterns, round to nearest even."""
    u = np.ascontiguousarray(a.astype(np.float32)).view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def quant_params(scales, offsets=None, signed=True):
    """fp32 scale bits in [31:0] (the unit keeps [31:13]), 9-bit offset at [45:37], sign flag at bit 46."""
    q = np.ascontiguousarray(scales.astype(np.float32)).view(np.uint32).astype(np.uint64)
    if offsets is not None:
        q |= (offsets.astype(np.int64) & 0x1FF).astype(np.uint64) << np.uint64(37)
    if signed:
        q |= np.uint64(1) << np.uint64(46)
    return q


def out_to_f32(bits, dtype):
    if dtype == ab.F32:
        return bits
    return orc.f16_bits_to_f32(bits) if dtype == ab.F16 else orc.bf16_bits_to_f32(bits)


NP_OUT = {ab.F32: np.float32, ab.F16: np.uint16, ab.BF16: np.uint16, ab.S8: np.int8, ab.S32: np.int32}


def mx_quantize(x, chunk=512):
    """fp32 [R,K] -> (packed e2m1 bytes [R,K/2], e8m0 scales [R,K/32]): per 32-element block
    e = floor(log2(amax)) - 2, scale byte = clamp(e+127, 0, 254), elements rounded to nearest
    (ties to the even code) on the e2m1 grid {0,.5,1,1.5,2,3,4,6} with saturation at +-6; even
    index in the low nibble.  (An OCP-MX style quantiser; the reference generator only draws random
    operands and scale bytes 127..129.)"""
    R, K = x.shape
    packed = np.empty((R, K // 2), np.uint8)
    sb = np.empty((R, K // 32), np.uint8)
    for r0 in range(0, R, chunk):
        blk = x[r0:r0 + chunk].reshape(-1, K // 32, 32).astype(np.float32)
        amax = np.abs(blk).max(axis=2)
        e = np.where(amax > 0, np.floor(np.log2(np.maximum(amax, 1e-38))) - 2, -127).astype(np.int32)
        s = np.clip(e + 127, 0, 254).astype(np.uint8)
        scaled = blk / np.exp2(s.astype(np.float32) - 127)[:, :, None]
        mag = np.abs(scaled)
        # midpoints of the grid; a tie goes to the neighbour with the even code
        idx = ((mag > 0.25).astype(np.uint8) + (mag >= 0.75) + (mag > 1.25) + (mag >= 1.75) + (mag > 2.5) + (mag >= 3.5) + (mag > 5.0))
        code = (idx | ((scaled < 0).astype(np.uint8) << 3)).astype(np.uint8).reshape(-1, K)
        packed[r0:r0 + chunk] = code[:, 0::2] | (code[:, 1::2] << 4)
        sb[r0:r0 + chunk] = s
    return packed, sb
