"""Helpers of the GPU tests: run a case through the C ABI on device buffers."""
import numpy as np

import cases

OPC = {"N": 1, "T": 2}


def torch_dt(dt):
    import torch
    return torch.float32 if dt == "f32" else torch.float64


def guard_alloc(n, dt, device="cuda", guard=256, fill=float("nan")):
    """Device buffer of n elements with poison bands on both sides; returns (view, whole)."""
    import torch
    whole = torch.full((n + 2 * guard,), 12345.0, dtype=torch_dt(dt), device=device)
    view = whole[guard:guard + n]
    view.fill_(fill)
    return view, whole


def guards_intact(whole, n, guard=256):
    return bool((whole[:guard] == 12345.0).all().item() and (whole[guard + n:] == 12345.0).all().item())


def run_case(h, c, use_temp2=True, x=None, fs=None, y=None, guard=True):
    """Execute case c on the GPU through {s,d}ge{mkm,kmm}; returns Z as a numpy array."""
    import torch
    if x is None:
        x, fs, y = cases.operands(c)
    tdt = torch_dt(c["dt"])
    K = int(np.prod(c["ps"], dtype=object))
    L = int(np.prod(c["qs"], dtype=object))
    M = c["M"]
    xd = torch.from_numpy(x).cuda()
    fd = [torch.from_numpy(f).cuda() for f in fs]
    yd = torch.from_numpy(y).cuda() if y is not None else None
    ye, te = h.sizes(M, c["ps"], c["qs"])
    assert ye == M * L
    z, zw = guard_alloc(ye, c["dt"])
    t1, t1w = guard_alloc(te, c["dt"])
    if use_temp2:
        t2, t2w = guard_alloc(te, c["dt"])
    else:
        # without temp2 the library may use Z as scratch, so Z must be as large as a temp
        z, zw = guard_alloc(max(ye, te), c["dt"])
        t2, t2w = None, None
    xcopy = xd.clone()
    h.raw_gemm(c["mm"], "s" if c["dt"] == "f32" else "d", M, c["ps"], c["qs"], xd.data_ptr(), OPC[c["opx"]],
               [f.data_ptr() for f in fd], OPC[c["opf"]], z.data_ptr(), c["alpha"], c["beta"],
               yd.data_ptr() if yd is not None else 0, t1.data_ptr(), t2.data_ptr() if t2 is not None else 0)
    torch.cuda.synchronize()
    if guard:
        assert guards_intact(zw, z.numel()), "write outside Z"
        assert guards_intact(t1w, te), "write outside temp1"
        if t2w is not None:
            assert guards_intact(t2w, te), "write outside temp2"
        assert torch.equal(xd, xcopy), "X was modified"
    out = z[:ye].cpu().numpy()
    return out.reshape((M, L) if c["mm"] == "mkm" else (L, M))
