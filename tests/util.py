import torch


def cos(a, b):
    a, b = a.double().flatten(), b.double().flatten()      # fp32 sums over millions of elements lose ~1e-4
    return float(torch.dot(a, b) / (a.norm() * b.norm() + 1e-30))


def assert_close(got, want, cos_min=0.9999, rel=0.005, abs_=1e-3, name=""):
    """The reference's golden criterion: cosine >= 0.9999 and max|d| <= rel*max|want| + abs."""
    g, w = got.float(), want.float()
    c = cos(g, w)
    md = float((g - w).abs().max())
    lim = rel * float(w.abs().max()) + abs_
    assert c >= cos_min and md <= lim, f"{name}: cos={c:.6f} max|d|={md:.5g} limit={lim:.5g}"
