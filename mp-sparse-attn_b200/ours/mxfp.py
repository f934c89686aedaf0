"""Host-side helpers for OCP microscaling element types, API-compatible with ours/mxfp.py of the
reference (MXFP4Tensor :12-236, MXScaleTensor :239-307).  Pure tensor arithmetic on whatever
device the data lives on; these are packing utilities, not part of the kernel path."""
import torch

_E2M1_MAGNITUDES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
# midpoints between consecutive magnitudes; a tie goes to the neighbour with mantissa bit 0
_E2M1_MIDPOINTS = ((0.25, False), (0.75, True), (1.25, False), (1.75, True), (2.5, False), (3.5, True), (5.0, False))


class MXFP4Tensor:
    """Four-bit E2M1 data, one code (S<<3 | E<<1 | M) per uint8."""

    def __init__(self, data=None, size=None, device=None, dtype=torch.float32):
        self.device = device
        if data is not None:
            assert isinstance(data, torch.Tensor), "Parameter data must be a torch tensor"
            self.device = data.device
            assert dtype in [torch.float32, torch.uint8], "Currently only float32 and uint8 are supported for fp4e2m1"
            self.data = self._from_float(data) if dtype == torch.float32 else self._from_uint8(data)
        elif size is not None:
            self.size = size if isinstance(size, tuple) else (size, )
        else:
            raise ValueError("Either parameter data or size must be provided")

    def random(self):
        self.data = torch.randint(0, 16, size=self.size, dtype=torch.uint8, device=self.device)
        return self

    def to(self, dtype):
        assert dtype == torch.float32, "Currently only float32 is supported for fp4e2m1 to float conversion"
        lut = torch.tensor(_E2M1_MAGNITUDES, dtype=torch.float32, device=self.data.device)
        code = self.data.to(torch.int64)
        mag = lut[code & 7]
        return torch.where((code & 8) != 0, -mag, mag)

    def _from_uint8(self, data):
        assert data.dtype == torch.uint8, "data must be uint8, but got {}".format(data.dtype)
        return data

    def _from_float(self, values):
        """float -> E2M1, round to nearest even, saturating; NaN/Inf saturate; zeros keep their sign."""
        sign = torch.signbit(values).to(torch.uint8)
        a = values.abs().to(torch.float32)
        a = torch.where(torch.isfinite(a), a, torch.full_like(a, _E2M1_MAGNITUDES[-1]))
        idx = torch.zeros(a.shape, dtype=torch.uint8, device=a.device)
        for mid, tie_up in _E2M1_MIDPOINTS:
            idx += ((a >= mid) if tie_up else (a > mid)).to(torch.uint8)
        return (sign << 3) | idx

    def to_packed_tensor(self, dim):
        """Two codes per byte along `dim`, even index in the low nibble; odd sizes are zero padded."""
        data = self.data
        assert 0 <= dim < data.ndim, "The dimension to pack along is not within the range of tensor dimensions"
        d = data.movedim(dim, -1)
        if d.shape[-1] % 2:
            d = torch.nn.functional.pad(d, (0, 1))
        packed = (d[..., 1::2] << 4) | d[..., 0::2]
        return packed.movedim(-1, dim).contiguous()

    def unpack_packed_tensor(self, packed_tensor, dim, original_shape):
        p = packed_tensor.movedim(dim, -1)
        both = torch.stack((p & 0xF, (p >> 4) & 0xF), dim=-1).flatten(-2)
        both = both[..., :original_shape[dim]]
        return both.movedim(-1, dim).contiguous().type(torch.uint8)


class MXScaleTensor:
    """E8M0 block scale factors: value 2^(code-127), code 255 = NaN."""

    def __init__(self, data=None, size=None, device=None):
        self.device = device
        if data is not None:
            assert isinstance(data, torch.Tensor), "Parameter data must be a torch tensor"
            self.device = data.device
            self.data = self._from_float(data)
        elif size is not None:
            self.size = size if isinstance(size, tuple) else (size, )
        else:
            raise ValueError("Either parameter data or size must be provided")

    def random(self, low=None, high=None):
        lo = 0 if low is None else max(0, int(torch.log2(torch.tensor(low))) + 127)
        hi = 254 if high is None else min(254, max(0, int(torch.log2(torch.tensor(high))) + 127))
        assert lo <= hi, "Low must be less than or equal to high"
        self.data = torch.randint(lo, hi + 1, size=self.size, dtype=torch.uint8, device=self.device)
        return self

    def to(self, dtype):
        assert dtype == torch.float32, "Currently only float32 is supported for f8e8m0 to float conversion"
        e = self.data.to(torch.float32)
        v = torch.exp2(e - 127.0)
        return torch.where(self.data == 255, torch.full_like(v, float("nan")), v)

    def _from_float(self, values):
        v = values.to(torch.float32)
        bad = ~torch.isfinite(v) | (v <= 0)
        e = torch.floor(torch.log2(torch.where(bad, torch.ones_like(v), v))) + 127.0
        e = e.to(torch.int32).clamp(0, 254).to(torch.uint8)
        return torch.where(bad, torch.full_like(e, 255), e)
