"""The training step on explicit samples restated with oracle calls only (CPU): the checker of
3dmaker_b200.pipeline.SampleTrainer and the body of the benchmark's CPU baseline."""
import numpy as np

import oracle as orc


class OracleField:
    def __init__(self, L, T, base, growth, scales, dls, density_dims, color_dims, table_f32, dW, db, cW, cb, scatter_scales=None):
        self.L, self.T, self.scales, self.dls = L, T, np.asarray(scales, np.float32), dls
        # the reference scatters with its own expression of the level resolutions (a few ulp from the forward's)
        self.scatter_scales = self.scales if scatter_scales is None else np.asarray(scatter_scales, np.float32)
        self.density_dims, self.color_dims = density_dims, color_dims
        self.table = np.ascontiguousarray(table_f32, np.float32).ravel().copy()
        self.dW, self.db, self.cW, self.cb = (np.asarray(a, np.float32).copy() for a in (dW, db, cW, cb))

    def forward_backward(self, pos4, dirs3, target_h8, loss_scale, density_bias=0.0):
        n = pos4.shape[0]
        th = orc.half_bits(self.table)
        enc = orc.encode_forward(pos4, th, self.scales, self.T, self.dls)
        d_out, d_acts = orc.mlp_forward(enc, self.density_dims, orc.half_bits(self.dW), self.db, save_acts=True)
        c_in, sigma = orc.sh_gather(dirs3, np.arange(n, dtype=np.uint32), d_out, density_bias)
        c_out, c_acts = orc.mlp_forward(c_in, self.color_dims, orc.half_bits(self.cW), self.cb, out_act=1, save_acts=True)
        total, c_grad = orc.mse_loss_grad(c_out, target_h8, 3, loss_scale, out_act=1)
        g_cW, g_cb, c_dx = orc.mlp_backward(c_grad, self.color_dims, orc.half_bits(self.cW), c_in, c_acts, want_dx=True)
        d_grad = orc.density_grad(np.zeros(n, np.float32), c_dx)
        g_dW, g_db, d_enc = orc.mlp_backward(d_grad, self.density_dims, orc.half_bits(self.dW), enc, d_acts, want_dx=True)
        g_table = orc.scatter_backward(pos4, d_enc, self.scatter_scales, self.T, self.dls)
        return dict(loss_sum=total, enc=enc, d_out=d_out, c_in=c_in, c_out=c_out, c_grad=c_grad, c_dx=c_dx, d_grad=d_grad,
                    d_enc=d_enc, g_table=g_table, g_dW=g_dW, g_db=g_db, g_cW=g_cW, g_cb=g_cb, sigma=sigma)


def oracle_ray_step(field, march, dirs3, rgb_true, bg, lambda_dist, loss_scale, density_bias, total_rays):
    """Everything of one NeRF optimizer step after the march, restated with oracle calls.
    march = dict(num_steps, ray_offsets, ray_indices, t, pos4) for the rays of the step (ray order)."""
    cnt, off, ridx, t, pos4 = (march[k] for k in ("num_steps", "ray_offsets", "ray_indices", "t", "pos4"))
    R, n = len(cnt), len(t)
    th = orc.half_bits(field.table)
    enc = orc.encode_forward(pos4, th, field.scales, field.T, field.dls)
    d_out, d_acts = orc.mlp_forward(enc, field.density_dims, orc.half_bits(field.dW), field.db, save_acts=True)
    c_in, sigma = orc.sh_gather(dirs3, ridx, d_out, density_bias)
    c_out, c_acts = orc.mlp_forward(c_in, field.color_dims, orc.half_bits(field.cW), field.cb, out_act=1, save_acts=True)
    rgb, depth, phi, dw, wsum = orc.render_rays_distortion(R, off, cnt, t, sigma, c_out[:, :3].copy(), rgb_true, lambda_dist, 0.0, bg)
    c_grad, dsig = orc.color_grad(R, cnt, off, t, d_out, c_out, phi, rgb, dw, wsum, loss_scale, density_bias, total_rays, grad_stride=8)
    g_cW, g_cb, c_dx = orc.mlp_backward(c_grad, field.color_dims, orc.half_bits(field.cW), c_in, c_acts, want_dx=True)
    d_grad = orc.density_grad(dsig, c_dx)
    g_dW, g_db, d_enc = orc.mlp_backward(d_grad, field.density_dims, orc.half_bits(field.dW), enc, d_acts, want_dx=True)
    g_table = orc.scatter_backward(pos4, d_enc, field.scatter_scales, field.T, field.dls)
    return dict(d_out=d_out, sigma=sigma, c_in=c_in, c_out=c_out, rgb=rgb, phi=phi, dw=dw, wsum=wsum, c_grad=c_grad, dsig=dsig, d_grad=d_grad,
                g_table=g_table, g_dW=g_dW, g_db=g_db, g_cW=g_cW, g_cb=g_cb)
