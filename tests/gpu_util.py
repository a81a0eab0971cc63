"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def host(t):
    return t.detach().cpu().numpy()


def block_inputs(orc, seed, n, h, w, c, k, gamma_sigma=0.2):
    """Seeded inputs of one Conv3x3+BN+ReLU block and its forward by the oracle."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n, h, w, c)).astype(np.float16)
    wt = (rng.standard_normal((k, 3, 3, c)) * np.sqrt(2.0 / (9 * c))).astype(np.float16)
    gamma = (1.0 + gamma_sigma * rng.standard_normal(k)).astype(np.float32)
    beta = (gamma_sigma * rng.standard_normal(k)).astype(np.float32)
    dy = rng.standard_normal((n, h, w, k)).astype(np.float16)
    fwd = orc.cbr_fwd_amp(x, wt, gamma, beta)
    return dict(x=x, w=wt, gamma=gamma, beta=beta, dy=dy, **fwd)
