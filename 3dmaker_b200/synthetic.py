"""Synthetic analytic scenes standing in for captured datasets (the reference's nerf_synthetic-style data is
not available): cameras, pinhole rays and ground-truth colours by numerical ray integration.

This is data generation, outside the timed hot path; it uses torch tensor maths on whatever device the
caller asks for.  Conventions follow the reference's camera code so rendered frames are comparable:
pinhole rays of generate_custom_rays_kernel (modules/NeRF/NerfTrainer.cu:25-47) and the orbit camera basis of
INerfTrainer::renderOrbit (NerfTrainer.cu:330-366).  The world is centred on the origin because the marcher
needs an AABB that straddles it (get_cascade divides by both bounds, modules/NeRF/processRays.cu:11-19).
"""
import math

import numpy as np


class SoftSphereScene:
    """density = 50 * sigmoid(-40 * (|x| - 0.3)), colour = x + 0.5, inside the box [-0.5, 0.5]^3."""
    aabb = 0.5

    def density(self, torch, x):
        return 50.0 * torch.sigmoid(-40.0 * (x.norm(dim=-1) - 0.3))

    def color(self, torch, x):
        return (x + 0.5).clamp(0.0, 1.0)


class MultiSphereScene:
    """32 seeded soft spheres (radii U[0.02, 0.15], random colours) in a box of half-extent `aabb * scale / 2`."""

    def __init__(self, n=32, seed=5, aabb=0.5, scale=4.0):
        rng = np.random.default_rng(seed)
        self.aabb = aabb
        self.extent = aabb * scale
        self.centers = rng.uniform(-self.extent * 0.8, self.extent * 0.8, size=(n, 3)).astype(np.float32)
        self.radii = rng.uniform(0.02, 0.15, size=n).astype(np.float32) * scale
        self.colors = rng.random((n, 3)).astype(np.float32)

    def _terms(self, torch, x):
        c = torch.as_tensor(self.centers, device=x.device)
        r = torch.as_tensor(self.radii, device=x.device)
        d = (x[..., None, :] - c).norm(dim=-1)
        return 50.0 * torch.sigmoid(-40.0 * (d - r))

    def density(self, torch, x):
        return self._terms(torch, x).sum(dim=-1)

    def color(self, torch, x):
        w = self._terms(torch, x)
        col = torch.as_tensor(self.colors, device=x.device)
        return (w[..., None] * col).sum(dim=-2) / w.sum(dim=-1, keepdim=True).clamp_min(1e-6)


def orbit_c2w(azimuth_deg, elevation_deg, radius, center=(0.0, 0.0, 0.0), up=(0.0, 1.0, 0.0)):
    """3x4 camera-to-world of the orbit camera (row-major), looking at `center`."""
    up = np.asarray(up, np.float64); up = up / np.linalg.norm(up)
    ref = np.array([0.0, 1.0, 0.0]) if abs(up[1]) < 0.9 else np.array([1.0, 0.0, 0.0])
    a = np.cross(up, ref); a /= np.linalg.norm(a)
    b = np.cross(up, a)
    az, el = math.radians(azimuth_deg), math.radians(elevation_deg)
    planar = math.cos(az) * a + math.sin(az) * b
    direction = math.cos(el) * planar + math.sin(el) * up
    eye = np.asarray(center, np.float64) + radius * direction
    f = np.asarray(center, np.float64) - eye; f /= np.linalg.norm(f)
    r = np.cross(f, up); r /= np.linalg.norm(r)
    u = np.cross(r, f)
    return np.stack([np.array([r[i], u[i], -f[i], eye[i]]) for i in range(3)]).astype(np.float32)


def sphere_cameras(n, radius=1.5):
    """n camera poses on a sphere (Fibonacci lattice, no seed), as (azimuth, elevation) orbit cameras."""
    poses = []
    golden = math.pi * (3.0 - math.sqrt(5.0))
    for i in range(n):
        y = 1.0 - 2.0 * (i + 0.5) / n
        el = math.degrees(math.asin(max(-0.98, min(0.98, y))))
        az = math.degrees((i * golden) % (2 * math.pi))
        poses.append(orbit_c2w(az, el, radius))
    return np.stack(poses)


def focal_from_fov(width, fov_deg):
    return 0.5 * width / math.tan(0.5 * math.radians(fov_deg))


def pixel_rays(torch, c2w, px, py, width, height, focal):
    """Rays through pixel centres (px, py) of cameras c2w [n, 3, 4] (one pose per ray or a single pose)."""
    dx = (px - width * 0.5) / focal
    dy = -(py - height * 0.5) / focal
    dz = -torch.ones_like(dx)
    d = torch.stack([dx, dy, dz], dim=-1)
    d = d / d.norm(dim=-1, keepdim=True)
    rot, org = c2w[..., :3], c2w[..., 3]
    dirs = (rot * d[..., None, :]).sum(dim=-1)
    return org.expand_as(dirs).contiguous().float(), dirs.contiguous().float()


def frame_rays(torch, c2w, width, height, fov_deg, device="cuda"):
    idx = torch.arange(width * height, device=device)
    px, py = (idx % width).float(), (idx // width).float()
    pose = torch.as_tensor(c2w, device=device)
    return pixel_rays(torch, pose, px, py, width, height, focal_from_fov(width, fov_deg))


def random_training_rays(torch, poses, n_rays, width, height, fov_deg, seed, device="cuda"):
    """n_rays random pixels of random cameras (seeded)."""
    g = torch.Generator(device=device); g.manual_seed(seed)
    cam = torch.randint(0, poses.shape[0], (n_rays,), generator=g, device=device)
    px = torch.randint(0, width, (n_rays,), generator=g, device=device).float()
    py = torch.randint(0, height, (n_rays,), generator=g, device=device).float()
    c2w = torch.as_tensor(poses, device=device)[cam]
    return pixel_rays(torch, c2w, px, py, width, height, focal_from_fov(width, fov_deg))


def ground_truth(torch, scene, rays_o, rays_d, bg, extent=None, steps=384, chunk=1 << 18):
    """Composited colour of every ray by midpoint quadrature inside the scene box (fp32 on the device, 384 steps:
    the integrand is smooth on the scale of box / 384)."""
    extent = scene.aabb if extent is None else extent
    out = torch.empty((rays_o.shape[0], 3), device=rays_o.device)
    bgc = torch.as_tensor(bg, device=rays_o.device, dtype=torch.float32)
    for s in range(0, rays_o.shape[0], chunk):
        o, d = rays_o[s:s + chunk], rays_d[s:s + chunk]
        inv = 1.0 / torch.where(d.abs() < 1e-8, torch.full_like(d, 1e-8), d)
        t1, t2 = (-extent - o) * inv, (extent - o) * inv
        near = torch.minimum(t1, t2).amax(dim=-1).clamp_min(0.0)
        far = torch.maximum(t1, t2).amin(dim=-1)
        hit = far > near
        dt = ((far - near).clamp_min(0.0) / steps)[:, None]
        t = near[:, None] + (torch.arange(steps, device=o.device)[None, :] + 0.5) * dt
        x = o[:, None, :] + t[..., None] * d[:, None, :]
        sigma = scene.density(torch, x) * hit[:, None]
        alpha = 1.0 - torch.exp(-sigma * dt)
        trans = torch.cumprod(torch.cat([torch.ones_like(alpha[:, :1]), 1.0 - alpha], dim=1), dim=1)
        w = alpha * trans[:, :-1]
        out[s:s + chunk] = (w[..., None] * scene.color(torch, x)).sum(dim=1) + trans[:, -1:] * bgc
    return out


def psnr(torch, pred, target):
    mse = ((pred - target) ** 2).mean().item()
    return -10.0 * math.log10(max(mse, 1e-12))
