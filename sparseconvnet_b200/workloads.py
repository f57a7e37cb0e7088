"""Seeded synthetic workloads and the networks they run through.

The reference is evaluated on handwriting, ShapeNet and ScanNet data that is not available
here; these generators stand in with the same shapes, sizes and sparsity patterns (voxelised
surfaces).  Sample `s` of configuration `c` always uses ``numpy.random.default_rng(1000*c+s)``,
so the CPU oracle and the GPU path see identical arrays.

  config 1  one SubmanifoldConvolution 3-D f3 32->32, 256^3, shells + plane patches, batch 1
  config 2  2-D stroke classifier (VGG stack -> SparseToDense), batch 100, field 87x87
  config 3  3-D U-Net m=32 reps=2 planes 32..224 on 4096^3, rooms of box/cylinder surfaces
  config 4  3-D SparseResNet on 127^3 (128 is not reachable by size-3/stride-2 steps)
  config 5  4-D (3+1) stack 4 x (SC 64->64 f3, 81 offsets + BatchNormReLU), moving shells
"""
import numpy as np
import torch

# The generators need numpy only.  The network builders take the package that provides the modules
# (`scn`): this package by default, or the reference's own `sparseconvnet` -- the two build the same
# module tree with the same parameter names, so a state_dict moves between them.  This file can be
# loaded by path without importing the package (and with it the CUDA library).


def _rng(config, sample):
    return np.random.default_rng(1000 * config + sample)


def _dedup(coords):
    return np.unique(np.asarray(coords, dtype=np.int64), axis=0)


def _shell(centre, radius, lo, hi):
    """Voxels p with | |p - centre| - radius | < 0.5 inside the box [lo, hi)."""
    c = np.asarray(centre, dtype=np.float64)
    a = np.maximum(np.floor(c - radius - 1).astype(np.int64), lo)
    b = np.minimum(np.ceil(c + radius + 2).astype(np.int64), hi)
    if np.any(b <= a):
        return np.zeros((0, len(c)), dtype=np.int64)
    axes = [np.arange(a[d], b[d]) for d in range(len(c))]
    g = np.meshgrid(*axes, indexing="ij", sparse=True)
    d2 = sum((g[d] - c[d]) ** 2 for d in range(len(c)))
    mask = np.abs(np.sqrt(d2) - radius) < 0.5
    idx = np.nonzero(mask)
    return np.stack([axes[d][idx[d]] for d in range(len(c))], axis=1)


# ---- config 1 -----------------------------------------------------------------------------------

def cloud_config1(sample=0, size=256, n_shells=20, n_planes=4):
    rng = _rng(1, sample)
    parts = []
    for _ in range(n_shells):
        parts.append(_shell(rng.uniform(0, size, 3), rng.uniform(8, 60), np.zeros(3, np.int64),
                            np.full(3, size, np.int64)))
    for _ in range(n_planes):
        axis = int(rng.integers(0, 3))
        pos = int(rng.integers(0, size))
        o = rng.integers(0, size - 96, 2)
        u, v = np.meshgrid(np.arange(o[0], o[0] + 96), np.arange(o[1], o[1] + 96), indexing="ij")
        cols = [u.reshape(-1), v.reshape(-1)]
        cols.insert(axis, np.full(u.size, pos))
        parts.append(np.stack(cols, axis=1))
    coords = _dedup(np.concatenate(parts))
    feats = rng.standard_normal((coords.shape[0], 32)).astype(np.float32)
    return coords, feats


# ---- config 2 -----------------------------------------------------------------------------------

def _bresenham(p, q):
    x0, y0, x1, y1 = int(p[0]), int(p[1]), int(q[0]), int(q[1])
    dx, dy = abs(x1 - x0), -abs(y1 - y0)
    sx, sy = (1 if x0 < x1 else -1), (1 if y0 < y1 else -1)
    err = dx + dy
    pts = []
    while True:
        pts.append((x0, y0))
        if x0 == x1 and y0 == y1:
            break
        e2 = 2 * err
        if e2 >= dy:
            err += dy
            x0 += sx
        if e2 <= dx:
            err += dx
            y0 += sy
    return pts


def strokes_config2(sample):
    rng = _rng(2, sample)
    pts = []
    for _ in range(int(rng.integers(3, 9))):
        verts = rng.integers(0, 64, (int(rng.integers(4, 13)), 2))
        for a, b in zip(verts[:-1], verts[1:]):
            pts.extend(_bresenham(a, b))
    return _dedup(np.asarray(pts))


def batch_config2(samples):
    cs = []
    for j, s in enumerate(samples):
        c = strokes_config2(s)
        cs.append(np.concatenate([c, np.full((c.shape[0], 1), j, np.int64)], axis=1))
    coords = np.concatenate(cs)
    return coords, np.ones((coords.shape[0], 1), dtype=np.float32)


# ---- config 3 -----------------------------------------------------------------------------------

def _box_surface(lo, hi):
    """1-voxel shell of the axis-aligned box [lo, hi] (inclusive corners)."""
    parts = []
    for axis in range(3):
        others = [d for d in range(3) if d != axis]
        u, v = np.meshgrid(np.arange(lo[others[0]], hi[others[0]] + 1),
                           np.arange(lo[others[1]], hi[others[1]] + 1), indexing="ij")
        for pos in (lo[axis], hi[axis]):
            cols = [None, None, None]
            cols[axis] = np.full(u.size, pos)
            cols[others[0]] = u.reshape(-1)
            cols[others[1]] = v.reshape(-1)
            parts.append(np.stack(cols, axis=1))
    return np.concatenate(parts)


def _cylinder_surface(cx, cy, r, z0, z1):
    t = np.arange(0, 2 * np.pi, 0.5 / max(r, 1.0))
    ring = np.unique(np.stack([np.rint(cx + r * np.cos(t)), np.rint(cy + r * np.sin(t))], axis=1).astype(np.int64), axis=0)
    zs = np.arange(z0, z1 + 1)
    side = np.concatenate([np.repeat(ring, zs.size, axis=0), np.tile(zs, ring.shape[0])[:, None]], axis=1)
    u, v = np.meshgrid(np.arange(int(cx - r), int(cx + r) + 1), np.arange(int(cy - r), int(cy + r) + 1), indexing="ij")
    disc = np.stack([u.reshape(-1), v.reshape(-1)], axis=1)
    disc = disc[(disc[:, 0] - cx) ** 2 + (disc[:, 1] - cy) ** 2 <= r * r]
    top = np.concatenate([disc, np.full((disc.shape[0], 1), z1)], axis=1)
    return np.concatenate([side, top])


def room_config3(sample, target_voxels=200000, field=4096):
    """Floor, ceiling and four walls of a 6-12 m x 6-12 m x 2.5-3 m box at 2 cm voxels with
    10-30 box and cylinder surfaces inside.  Complete surfaces of such a room are 0.4-1 M
    voxels; like a real scan, which sees only part of every surface, the room is thinned to
    about `target_voxels` by keeping whole 8x8x8-voxel blocks chosen by a seeded draw, so the
    local surface structure (what the rulebooks see) is preserved."""
    rng = _rng(3, sample)
    ext = np.array([rng.integers(300, 601), rng.integers(300, 601), rng.integers(125, 151)])
    parts = [_box_surface(np.zeros(3, np.int64), ext - 1)]
    for _ in range(int(rng.integers(10, 31))):
        if rng.random() < 0.6:
            sz = np.array([rng.integers(20, 120), rng.integers(20, 120), rng.integers(20, 100)])
            lo = np.array([rng.integers(1, ext[0] - sz[0] - 1), rng.integers(1, ext[1] - sz[1] - 1), 1])
            parts.append(_box_surface(lo, lo + sz))
        else:
            r = float(rng.uniform(8, 40))
            cx = float(rng.uniform(r + 2, ext[0] - r - 2))
            cy = float(rng.uniform(r + 2, ext[1] - r - 2))
            parts.append(_cylinder_surface(cx, cy, r, 1, int(rng.integers(20, 110))))
    coords = _dedup(np.concatenate(parts))
    coords = coords[np.all((coords >= 0) & (coords < ext), axis=1)]
    if target_voxels and coords.shape[0] > target_voxels:
        keep_p = target_voxels / coords.shape[0]
        blk = coords // 8
        h = (blk[:, 0] * 73856093) ^ (blk[:, 1] * 19349663) ^ (blk[:, 2] * 83492791) ^ int(rng.integers(1 << 30))
        h = (h * 2654435761) & 0xFFFFFFFF
        coords = coords[(h / 4294967296.0) < keep_p]
    origin = np.array([rng.integers(0, field - ext[0]), rng.integers(0, field - ext[1]), rng.integers(0, field - ext[2])])
    coords = coords + origin
    feats = rng.uniform(-1, 1, (coords.shape[0], 3)).astype(np.float32)
    return coords, feats


def batch_config3(samples, target_voxels=200000):
    cs, fs = [], []
    for j, s in enumerate(samples):
        c, f = room_config3(s, target_voxels)
        cs.append(np.concatenate([c, np.full((c.shape[0], 1), j, np.int64)], axis=1))
        fs.append(f)
    return np.concatenate(cs), np.concatenate(fs)


# ---- config 4 -----------------------------------------------------------------------------------

def shape_config4(sample, size=127):
    """Surface voxels of a randomly rotated superquadric |x/a|^e1 + |y/b|^e2 + |z/c|^e3 = 1."""
    rng = _rng(4, sample)
    e = rng.uniform(0.3, 3.0, 3)
    sc = rng.uniform(20, 60, 3)
    q, _ = np.linalg.qr(rng.standard_normal((3, 3)))
    ax = np.arange(size) - (size - 1) / 2.0
    g = np.stack(np.meshgrid(ax, ax, ax, indexing="ij"), axis=-1) @ q
    f = sum(np.abs(g[..., d] / sc[d]) ** e[d] for d in range(3))
    inside = f < 1.0
    pad = np.pad(inside, 1, constant_values=False)
    core = inside.copy()
    for d in range(3):
        for sh in (0, 2):
            sl = [slice(1, -1)] * 3
            sl[d] = slice(sh, sh + size)
            core &= pad[tuple(sl)]
    return np.stack(np.nonzero(inside & ~core), axis=1).astype(np.int64)


def batch_config4(samples):
    cs = []
    for j, s in enumerate(samples):
        c = shape_config4(s)
        cs.append(np.concatenate([c, np.full((c.shape[0], 1), j, np.int64)], axis=1))
    coords = np.concatenate(cs)
    return coords, np.ones((coords.shape[0], 1), dtype=np.float32)


# ---- config 5 -----------------------------------------------------------------------------------

def sequence_config5(sample, size=256, frames=8, n_shells=5):
    rng = _rng(5, sample)
    centres = rng.uniform(60, size - 60, (n_shells, 3))
    radii = rng.uniform(20, 35, n_shells)
    vel = rng.uniform(1, 3, (n_shells, 3)) * rng.choice([-1.0, 1.0], (n_shells, 3))
    parts = []
    for t in range(frames):
        fr = [_shell(centres[i] + vel[i] * t, radii[i], np.zeros(3, np.int64), np.full(3, size, np.int64))
              for i in range(n_shells)]
        c = _dedup(np.concatenate(fr))
        parts.append(np.concatenate([c, np.full((c.shape[0], 1), t, np.int64)], axis=1))
    return np.concatenate(parts)


def batch_config5(samples):
    cs = []
    for j, s in enumerate(samples):
        c = sequence_config5(s)
        cs.append(np.concatenate([c, np.full((c.shape[0], 1), j, np.int64)], axis=1))
    coords = np.concatenate(cs)
    rng = _rng(5, 900 + int(samples[0]))
    return coords, rng.standard_normal((coords.shape[0], 64)).astype(np.float32)


# ---- networks --------------------------------------------------------------------------------------

def _default_package():
    import sparseconvnet_b200
    return sparseconvnet_b200


def randomize(model, seed):
    """Seeded non-trivial state: BatchNorm statistics and affine terms away from (0, 1) so a
    wrong mean/variance/eps convention cannot hide.  Convolution weights keep the module's own
    initialisation (drawn under the same seed)."""
    g = torch.Generator().manual_seed(seed)
    for m in model.modules():
        if hasattr(m, "running_mean") and hasattr(m, "nPlanes") and getattr(m, "weight", None) is not None:
            m.running_mean.copy_(torch.randn(m.nPlanes, generator=g) * 0.2)
            m.running_var.copy_(torch.rand(m.nPlanes, generator=g) + 0.5)
            m.weight.data.copy_(torch.rand(m.nPlanes, generator=g) + 0.5)
            m.bias.data.copy_(torch.randn(m.nPlanes, generator=g) * 0.2)
    return model


def build_config(config, seed=0, scn=None):
    """Returns (input_layer, sparse_model, head) for benchmark configuration 1..5; `head` is a
    torch.nn.Linear applied to `.features` or None.  Eval mode, seeded weights.  `scn` is the
    package the modules come from (default: sparseconvnet_b200)."""
    scn = scn or _default_package()
    torch.manual_seed(1234 + 17 * config + seed)
    head = None
    if config == 1:
        inp = scn.InputLayer(3, 256, mode=0)
        net = scn.Sequential().add(scn.SubmanifoldConvolution(3, 32, 32, 3, False))
    elif config == 2:
        net = scn.Sequential().add(
            scn.SparseVggNet(2, 1, [["C", 8], ["C", 8], ["MP", 3, 2], ["C", 16], ["C", 16], ["MP", 3, 2],
                                    ["C", 24], ["C", 24], ["MP", 3, 2]])).add(
            scn.SubmanifoldConvolution(2, 24, 32, 3, False)).add(scn.BatchNormReLU(32)).add(
            scn.SparseToDense(2, 32))
        inp = scn.InputLayer(2, net.input_spatial_size(torch.LongTensor([10, 10])), mode=3)
    elif config == 3:
        inp = scn.InputLayer(3, 4096, mode=4)
        net = scn.Sequential().add(scn.SubmanifoldConvolution(3, 3, 32, 3, False)).add(
            scn.UNet(3, 2, [32, 64, 96, 128, 160, 192, 224], False)).add(scn.BatchNormReLU(32))
        head = torch.nn.Linear(32, 20)
    elif config == 4:
        inp = scn.InputLayer(3, 127, mode=3)
        net = scn.Sequential().add(scn.SubmanifoldConvolution(3, 1, 16, 3, False)).add(
            scn.MaxPooling(3, 3, 2)).add(
            scn.SparseResNet(3, 16, [["b", 16, 2, 1], ["b", 32, 2, 2], ["b", 64, 2, 2], ["b", 128, 2, 2]]))
        head = torch.nn.Linear(128, 50)
    elif config == 5:
        inp = scn.InputLayer(4, [256, 256, 256, 8], mode=0)
        net = scn.Sequential()
        for _ in range(4):
            net.add(scn.SubmanifoldConvolution(4, 64, 64, 3, False)).add(scn.BatchNormReLU(64))
    else:
        raise ValueError("config must be 1..5")
    randomize(net, 99 + config + seed)
    net.eval()
    if head is not None:
        head.eval()
    return inp, net, head


def make_batch(config, samples):
    """(coords int64 [n, D+1 or D], features float32 [n, C]) for the given sample indices."""
    if config == 1:
        return cloud_config1(samples[0])
    return {2: batch_config2, 3: batch_config3, 4: batch_config4, 5: batch_config5}[config](list(samples))
