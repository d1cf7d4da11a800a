"""float64 autograd statement of the MoE block, independent of the C++ oracle.

Used only to check the oracle's hand-written backward: the same math in torch with
bf16 rounding points left out (they are straight-through for gradients)."""
import torch


def silu(x):
    return x * torch.sigmoid(x)


def moe_loss(X, Wr, Wup, Wdown, idx, dY, hidden, aux, zcoef, counts, bias=None):
    """Scalar whose gradients are what moe_backward returns: <Y, dY> + aux/z terms with the
    routing decision (idx) and the counts held constant (as the reference does)."""
    T, D = X.shape
    E = Wr.shape[0]
    K = idx.shape[1]
    logits = X @ Wr.t()
    if bias is not None:
        logits = logits + bias
    p = torch.softmax(logits, dim=1)
    psel = torch.gather(p, 1, idx)
    w = psel / psel.sum(1, keepdim=True)
    Y = torch.zeros(T, D, dtype=X.dtype)
    for j in range(K):
        for e in range(E):
            m = idx[:, j] == e
            if not m.any():
                continue
            x = X[m]
            if hidden > 0:
                o = silu(x @ Wup[e].t()) @ Wdown[e].t()
            else:
                o = silu(x @ Wup[e].t())
            Y[m] = Y[m] + w[m, j:j + 1] * o
    loss = (Y * dY).sum()
    if E > 1:
        lse = torch.logsumexp(logits, dim=1)
        f = counts.to(X.dtype) / (T * K)
        loss = loss + zcoef * (lse ** 2).sum() / T + aux * E / T * (p * f).sum()
    return loss, Y
