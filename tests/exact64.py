"""Float64 twins of the layers whose fp32 results are compared at a widened absolute tolerance. They are not the checker
(the fp32 restatement in oracle/ is): they measure how far an fp32 evaluation - the checker's or the GPU's - is from the
exact value, so that a test can show a widened tolerance absorbs fp32 rounding and nothing else."""
import numpy as np

F = np.float64


def _bc(v):
    return np.asarray(v, F)[None, :, None, None]


def act_fwd(name, v, slope):
    if name == "relu0":
        return np.where(v >= 0, v, 0.0)
    if name == "relu01":
        return np.where(v >= 0, v, v * F(np.float32(0.1)))
    if name == "prelu":
        return np.where(v >= 0, v, v * _bc(slope))
    if name == "elu":
        return np.where(v >= 0, v, np.expm1(np.minimum(v, 0.0)))
    if name == "tanh":
        return F(np.float32(1.7159)) * np.tanh(F(np.float32(0.6666)) * v)
    if name == "sigmoid":
        return 1.0 / (1.0 + np.exp(-v))
    raise ValueError(name)


def act_bwd(name, g, a_in, a_out, slope):
    """Gradient of the layer's input; the derivative in the form the reference uses (from the input for the rectifiers, from the
    output for the others)."""
    if name == "relu0":
        return np.where(a_in >= 0, g, 0.0)
    if name == "relu01":
        return np.where(a_in >= 0, g, g * F(np.float32(0.1)))
    if name == "prelu":
        return np.where(a_in >= 0, g, g * _bc(slope))
    if name == "elu":
        return np.where(a_out >= 0, g, g * (a_out + 1.0))
    if name == "tanh":
        sc, st = F(np.float32(1.7159)), F(np.float32(0.6666))
        return g * (sc * st) * (1.0 - (a_out / sc) ** 2)
    if name == "sigmoid":
        return g * a_out * (1.0 - a_out)
    raise ValueError(name)


def bn_train_chain(x, dy, gamma, beta, slope, chain, eps):
    """Training batch norm + activation chain and its backward pass in float64: y, saved {mean, invstd}, dx, u (the batch-norm output)."""
    xd, c = np.asarray(x, F), x.shape[1]
    mean = xd.mean(axis=(0, 2, 3))
    var = ((xd - _bc(mean)) ** 2).mean(axis=(0, 2, 3))
    inv = 1.0 / np.sqrt(var + F(np.float32(eps)))
    xh = (xd - _bc(mean)) * _bc(inv)
    u = xh * _bc(gamma) + _bc(beta)
    ins, v = [], u
    for name in chain:
        ins.append(v)
        v = act_fwd(name, v, slope)
    y = v
    g = np.asarray(dy, F)
    outs = ins[1:] + [y]
    for name, a_in, a_out in reversed(list(zip(chain, ins, outs))):
        g = act_bwd(name, g, a_in, a_out, slope)
    m = xd.size // c
    db, dg = g.sum(axis=(0, 2, 3)), (g * xh).sum(axis=(0, 2, 3))
    dx = _bc(np.asarray(gamma, F) * inv / m) * (m * g - _bc(db) - xh * _bc(dg))
    return y, np.concatenate([mean, inv]), dx, u


def softmax_bwd(dy, y, dx0=None):
    yd, dyd = np.asarray(y, F), np.asarray(dy, F)
    s = (yd * dyd).sum(axis=1, keepdims=True)
    dx = yd * (dyd - s)
    return dx if dx0 is None else dx + np.asarray(dx0, F)


def nll_fwd(p, t, mask=None, scale=1.0):
    pd, td = np.asarray(p, F), np.asarray(t, F)
    err = -(np.where(td > 0, td * np.log(np.maximum(pd, 1e-20)), 0.0)).sum(axis=1, keepdims=True) * F(np.float32(scale))
    return err if mask is None else err * np.asarray(mask, F)
