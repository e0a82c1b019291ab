"""A second, independent restatement of the network in vectorised float64 numpy, written from the
formulas rather than from the oracle's loops; the CPU tests check the C oracle against it."""
import numpy as np
from numpy.lib.stride_tricks import sliding_window_view


def split(params, F=6, P=6):
    S = F * P * P
    o = 0
    Wc = params[o:o + F * 25].reshape(F, 5, 5); o += F * 25
    bc = params[o:o + F]; o += F
    Ws = params[o:o + 16].reshape(4, 4); o += 16
    bs = params[o]; o += 1
    Wf = params[o:o + 10 * S].reshape(10, S); o += 10 * S
    bf = params[o:o + 10]
    return Wc, bc, Ws, bs, Wf, bf


def sig(v):
    return 1.0 / (1.0 + np.exp(-v))


def forward(params, x, H=28, F=6):
    params = np.asarray(params, dtype=np.float64)
    x = np.asarray(x, dtype=np.float64).reshape(H, H)
    C = H - 4
    P = C // 4
    Wc, bc, Ws, bs, Wf, bf = split(params, F, P)
    win = sliding_window_view(x, (5, 5))                      # [C, C, 5, 5]
    zc = np.einsum("yxij,fij->fyx", win, Wc) + bc[:, None, None]
    ac = sig(zc)
    blocks = ac[:, :4 * P, :4 * P].reshape(F, P, 4, P, 4)        # [f, p, i, q, j]
    zs = np.einsum("fpiqj,ij->fpq", blocks, Ws) + bs
    as_ = sig(zs)
    zf = Wf @ as_.reshape(-1) + bf
    af = sig(zf)
    return dict(x=x, zc=zc, ac=ac, zs=zs, as_=as_, zf=zf, af=af)


def gradient(params, x, label, H=28, F=6):
    """Per-image update direction (what one reference step adds, divided by dt), arena order."""
    params = np.asarray(params, dtype=np.float64)
    C = H - 4
    P = C // 4
    S = F * P * P
    Wc, bc, Ws, bs, Wf, bf = split(params, F, P)
    a = forward(params, x, H, F)
    df = -a["af"].copy()
    df[label] += 1.0
    gWf = np.outer(df, a["as_"].reshape(-1))
    das = (Wf.T @ df).reshape(F, P, P)
    ds = das * a["as_"] * (1 - a["as_"])
    blocks = a["ac"][:, :4 * P, :4 * P].reshape(F, P, 4, P, 4)
    gWs = np.einsum("fpq,fpiqj->ij", ds, blocks)
    gbs = ds.sum() / S
    dac = np.zeros_like(a["ac"])
    dac[:, :4 * P, :4 * P] = np.einsum("fpq,ij->fpiqj", ds, Ws).reshape(F, 4 * P, 4 * P)
    dc = dac * a["ac"] * (1 - a["ac"])
    win = sliding_window_view(a["x"], (5, 5))                 # [C, C, 5, 5]
    gWc = np.einsum("fyx,yxij->fij", dc, win) / (C * C)
    gbc = dc.sum(axis=(1, 2)) / (C * C)
    G = np.concatenate([gWc.reshape(-1), gbc, gWs.reshape(-1), [gbs], gWf.reshape(-1), df])
    return G, float(np.sqrt((df ** 2).sum())), dict(df=df, gWf=gWf, das=das, ds=ds, gWs=gWs, dac=dac, dc=dc, gWc=gWc)
