"""The named synthetic workloads (shapes, value distributions, neighbour targets) and their seeded
generation on the device.  Used by the benchmark and by the full-size parity tests, so that both run
on the same data.  Public datasets the reference was measured on are not available here; seeded
synthetic inputs with the same shapes and distributions stand in for them."""
from __future__ import annotations

import numpy as np

SEED = 2137834274  # the reference's dataset seed (source/DataLoader/ExponentialPointGenerator.hpp:11)

# name -> shape, distribution, target mean neighbours per point, epsilon (None: tuned at start-up
# with band joins through the library itself, like the reference's Python driver does with reRun).
WORKLOADS = {
    # the reference's own seeded `-e` stream (host generator, bit-identical to the reference's loader)
    "c1": dict(n=4096, d=128, dist="exp_ref", target=32, eps=0.3136),
    "c2": dict(n=100_000, d=384, dist="unit_gauss", target=16, eps=None),
    "c3": dict(n=1_000_000, d=4096, dist="exp", target=64, eps=None),
    "c4": dict(n=2_000_000, d=1024, dist="mixture", target=2000, eps=None, pairs_per_point=2600),
    "c5": dict(n=4_000_000, d=2048, dist="exp", target=8, eps=None),
}


def padded_dim(d: int) -> int:
    return -(-d // 64) * 64


def fill_device(sj, dev_pts, wl: dict) -> None:
    """Fill rows [0, n) of dev_pts (a CUDA float16 tensor of at least n rows, row stride = padded d,
    zero-initialised) with the workload's seeded data.  sj: a SelfJoin on the same device."""
    import torch
    n, d = wl["n"], wl["d"]
    ld = dev_pts.shape[1]
    kind = wl["dist"]
    # whatever produced dev_pts (its zero fill) ran on a torch stream; the library works on its own
    torch.cuda.current_stream(dev_pts.device).synchronize()
    if kind == "exp":
        # counter-based generator on the device: the reference's distribution (Exponential(40), rejected
        # to [0, 10], double -> float -> half), not its sequential stream
        sj.fill_exponential_device(dev_pts.data_ptr(), n, d, ld, 40.0, 10.0, SEED)
    elif kind == "exp_ref":
        from . import _lib
        host = _lib.dataset_exponential(n, d)
        dev_pts[:n, :d] = torch.from_numpy(host.view(np.float16)).to(dev_pts.device)
    elif kind == "unit_gauss":
        g = torch.Generator(device=dev_pts.device).manual_seed(SEED)
        for a in range(0, n, 65536):
            x = torch.randn((min(65536, n - a), d), generator=g, device=dev_pts.device, dtype=torch.float32)
            x /= x.norm(dim=1, keepdim=True)
            dev_pts[a:a + x.shape[0], :d] = x.to(torch.float16)
    elif kind == "mixture":
        # 256 centres ~ U[0,1]^D, cluster sizes ~ Zipf(1.1) over ranks 1..256 (largest remainder
        # rounding to sum N), point = centre + N(0, 0.05^2) per coordinate, points of a cluster contiguous
        g = torch.Generator(device=dev_pts.device).manual_seed(SEED)
        centres = torch.rand((256, d), generator=g, device=dev_pts.device, dtype=torch.float32)
        w = 1.0 / np.arange(1, 257) ** 1.1
        exact = w / w.sum() * n
        sizes = np.floor(exact).astype(np.int64)
        for i in np.argsort(-(exact - sizes))[: n - int(sizes.sum())]:
            sizes[i] += 1
        a = 0
        for cid, sz in enumerate(sizes):
            for b in range(0, int(sz), 65536):
                m = min(65536, int(sz) - b)
                x = centres[cid] + 0.05 * torch.randn((m, d), generator=g, device=dev_pts.device, dtype=torch.float32)
                dev_pts[a:a + m, :d] = x.to(torch.float16)
                a += m
    else:
        raise ValueError(kind)
    torch.cuda.current_stream(dev_pts.device).synchronize()


def host_sample(wl: dict, rows: int) -> np.ndarray:
    """Seeded host-side sample with the workload's distribution, binary16 bit patterns (rows, d)."""
    rng = np.random.default_rng(SEED)
    d = wl["d"]
    kind = wl["dist"]
    if kind in ("exp", "exp_ref"):
        x = np.minimum(rng.exponential(1.0 / 40.0, size=(rows, d)), 10.0)
    elif kind == "unit_gauss":
        x = rng.standard_normal((rows, d))
        x /= np.linalg.norm(x, axis=1, keepdims=True)
    elif kind == "mixture":
        centres = rng.uniform(0.0, 1.0, size=(256, d))
        w = 1.0 / np.arange(1, 257) ** 1.1
        x = centres[rng.choice(256, size=rows, p=w / w.sum())] + rng.normal(0.0, 0.05, size=(rows, d))
    else:
        raise ValueError(kind)
    return x.astype(np.float32).astype(np.float16).view(np.uint16)
