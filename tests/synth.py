"""Seeded synthetic inputs with the shapes and value distributions of the five benchmark
configurations (stand-ins: the reference ships no dataset for this path). Everything is generated on
the host with numpy so that the CPU checker and the GPU see identical bits; multi-GPU shards are
slices of the same full-batch tensor."""
import numpy as np


def rng(config_id, salt=0):
    return np.random.Generator(np.random.PCG64(1000 + config_id + 7919 * salt))


def normal(g, shape, mean=0.0, std=1.0):
    return (g.standard_normal(shape, dtype=np.float32) * np.float32(std) + np.float32(mean)).astype(np.float32)


def uniform(g, shape, lo, hi):
    return (g.random(shape, dtype=np.float32) * np.float32(hi - lo) + np.float32(lo)).astype(np.float32)


def bn_params(g, c, eps=1e-5):
    """gamma~U(0.5,1.5), beta~N(0,0.1), running mean~N(0,0.1), running var~U(0.5,2) -> invsigma.
    The reference's 4th weight chunk is the inverse standard deviation (nnforge/batch_norm_layer.h:26),
    so the variance is converted on the host."""
    gamma = uniform(g, c, 0.5, 1.5)
    beta = normal(g, c, 0.0, 0.1)
    mean = normal(g, c, 0.0, 0.1)
    var = uniform(g, c, 0.5, 2.0)
    invsigma = (1.0 / np.sqrt(var.astype(np.float64) + eps)).astype(np.float32)
    return gamma, beta, mean, invsigma


def edge_values():
    """Values every elementwise test mixes in: signed zeros, denormals, infinities, huge/small."""
    return np.array([0.0, -0.0, 1e-45, -1e-45, 1e-38, -1e-38, np.inf, -np.inf, 3.4e38, -3.4e38, 1.0, -1.0, 88.0, -88.0, 20.0, -20.0],
                    dtype=np.float32)


def with_edges(g, a):
    a = a.copy()
    flat = a.reshape(-1)
    ev = edge_values()
    if flat.size >= 4 * ev.size:
        pos = g.choice(flat.size, ev.size, replace=False)
        flat[pos] = ev
    return a


def targets(g, shape, soft_entries=1):
    """Dense target tensor [N,C,H,W] for a loss over channels: one-hot labels per (entry, pixel); the first
    `soft_entries` entries carry soft targets (random non-negative weights, about half of them zero)."""
    n, c = shape[0], shape[1]
    t = np.zeros(shape, np.float32)
    labels = g.integers(0, c, size=(n,) + tuple(shape[2:]))
    np.put_along_axis(t, labels[:, None], 1.0, axis=1)
    for e in range(min(soft_entries, n)):
        w = g.random(shape[1:], dtype=np.float32)
        t[e] = w * (g.random(shape[1:]) > 0.5)
    return t
