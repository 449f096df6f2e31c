"""float64 numpy references for the contractions whose parity the reference's own tests do not pin
(conv2d, conv2d_transpose, max_pool2d): direct definitions, no shared code with the oracle or the
CUDA kernels."""
import numpy as np


def conv2d(x, w, b, stride, pad):
    x = x.astype(np.float64); w = w.astype(np.float64)
    n, cin, h, wd = x.shape
    cout, _, kh, kw = w.shape
    sh, sw = stride; ph, pw = pad
    ho = (h + 2 * ph - kh) // sh + 1
    wo = (wd + 2 * pw - kw) // sw + 1
    xp = np.zeros((n, cin, h + 2 * ph, wd + 2 * pw)); xp[:, :, ph:ph + h, pw:pw + wd] = x
    y = np.zeros((n, cout, ho, wo))
    for ky in range(kh):
        for kx in range(kw):
            patch = xp[:, :, ky:ky + (ho - 1) * sh + 1:sh, kx:kx + (wo - 1) * sw + 1:sw]
            y += np.einsum("nchw,oc->nohw", patch, w[:, :, ky, kx])
    if b is not None:
        y += b.astype(np.float64)[None, :, None, None]
    return y


def conv2d_backward(x, w, g, stride, pad):
    x = x.astype(np.float64); w = w.astype(np.float64); g = g.astype(np.float64)
    n, cin, h, wd = x.shape
    cout, _, kh, kw = w.shape
    sh, sw = stride; ph, pw = pad
    ho, wo = g.shape[2], g.shape[3]
    xp = np.zeros((n, cin, h + 2 * ph, wd + 2 * pw)); xp[:, :, ph:ph + h, pw:pw + wd] = x
    dxp = np.zeros_like(xp)
    dw = np.zeros_like(w)
    for ky in range(kh):
        for kx in range(kw):
            sl = (slice(None), slice(None), slice(ky, ky + (ho - 1) * sh + 1, sh), slice(kx, kx + (wo - 1) * sw + 1, sw))
            dw[:, :, ky, kx] = np.einsum("nohw,nchw->oc", g, xp[sl])
            dxp[sl] += np.einsum("nohw,oc->nchw", g, w[:, :, ky, kx])
    return dxp[:, :, ph:ph + h, pw:pw + wd], dw, g.sum(axis=(0, 2, 3))


def conv2d_transpose(x, w, b, stride, pad):
    x = x.astype(np.float64); w = w.astype(np.float64)
    n, cin, h, wd = x.shape
    _, cout, kh, kw = w.shape
    sh, sw = stride; ph, pw = pad
    oh = (h - 1) * sh + kh - 2 * ph
    ow = (wd - 1) * sw + kw - 2 * pw
    full = np.zeros((n, cout, (h - 1) * sh + kh, (wd - 1) * sw + kw))
    for ky in range(kh):
        for kx in range(kw):
            full[:, :, ky:ky + (h - 1) * sh + 1:sh, kx:kx + (wd - 1) * sw + 1:sw] += np.einsum("nchw,co->nohw", x, w[:, :, ky, kx])
    y = full[:, :, ph:ph + oh, pw:pw + ow].copy()
    if b is not None:
        y += b.astype(np.float64)[None, :, None, None]
    return y


def conv2d_transpose_backward(x, w, g, stride, pad):
    x = x.astype(np.float64); w = w.astype(np.float64); g = g.astype(np.float64)
    n, cin, h, wd = x.shape
    _, cout, kh, kw = w.shape
    sh, sw = stride; ph, pw = pad
    gfull = np.zeros((n, cout, (h - 1) * sh + kh, (wd - 1) * sw + kw))
    gfull[:, :, ph:ph + g.shape[2], pw:pw + g.shape[3]] = g
    dx = np.zeros_like(x); dw = np.zeros_like(w)
    for ky in range(kh):
        for kx in range(kw):
            gs = gfull[:, :, ky:ky + (h - 1) * sh + 1:sh, kx:kx + (wd - 1) * sw + 1:sw]
            dx += np.einsum("nohw,co->nchw", gs, w[:, :, ky, kx])
            dw[:, :, ky, kx] = np.einsum("nchw,nohw->co", x, gs)
    return dx, dw, g.sum(axis=(0, 2, 3))


def max_pool2d(x, k, s, p):
    n, c, h, w = x.shape
    ho = (h + 2 * p[0] - k[0]) // s[0] + 1
    wo = (w + 2 * p[1] - k[1]) // s[1] + 1
    y = np.full((n, c, ho, wo), -np.inf, dtype=np.float32)
    idx = np.zeros((n, c, ho, wo), dtype=np.float32)
    for yo in range(ho):
        for xo in range(wo):
            best = np.full((n, c), -np.inf, dtype=np.float32); bi = np.zeros((n, c), dtype=np.float32)
            i = 0
            for ky in range(k[0]):
                for kx in range(k[1]):
                    iy, ix = yo * s[0] + ky - p[0], xo * s[1] + kx - p[1]
                    if 0 <= iy < h and 0 <= ix < w:
                        v = x[:, :, iy, ix]
                        m = v > best
                        best = np.where(m, v, best); bi = np.where(m, np.float32(i), bi)
                    i += 1
            y[:, :, yo, xo] = best; idx[:, :, yo, xo] = bi
    return y, idx
