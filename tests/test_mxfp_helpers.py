"""ours.mxfp helper classes against golden vectors from the reference's ours/mxfp.py."""
import os

import numpy as np
import torch

from ours.mxfp import MXFP4Tensor, MXScaleTensor

G = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_mxfp4_tensor_matches_reference():
    z = np.load(os.path.join(G, "mxfp_helpers.npz"))
    vals = torch.from_numpy(z["fp4_in"])
    t = MXFP4Tensor(data=vals.clone())
    assert np.array_equal(t.data.numpy(), z["fp4_codes"])
    packed = t.to_packed_tensor(dim=0)
    assert np.array_equal(packed.numpy(), z["fp4_packed"])
    assert np.array_equal(t.unpack_packed_tensor(packed, 0, t.data.shape).numpy(), z["fp4_unpacked"])
    dec = MXFP4Tensor(data=torch.arange(16, dtype=torch.uint8), dtype=torch.uint8).to(torch.float32)
    assert np.array_equal(dec.numpy(), z["fp4_decode16"])
    # packing along an inner dimension of a 3-D tensor, odd length
    x = MXFP4Tensor(size=(2, 5, 3)).random()
    p = x.to_packed_tensor(dim=1)
    assert p.shape == (2, 3, 3)
    assert torch.equal(x.unpack_packed_tensor(p, 1, x.data.shape), x.data)


def test_mxscale_tensor_matches_reference():
    z = np.load(os.path.join(G, "mxfp_helpers.npz"))
    st = MXScaleTensor(data=torch.from_numpy(z["e8m0_in"]))
    assert np.array_equal(st.data.numpy(), z["e8m0_codes"])
    d = MXScaleTensor(size=(256,))
    d.data = torch.arange(256, dtype=torch.int32).to(torch.uint8)
    out = d.to(torch.float32).numpy()
    assert np.isnan(out[255]) and np.array_equal(out[:255], z["e8m0_decode256"][:255])
    r = MXScaleTensor(size=(64,)).random(low=0.5, high=8.0)
    assert int(r.data.min()) >= 126 and int(r.data.max()) <= 130
