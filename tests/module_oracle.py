"""The layer modules restated with the oracle operators (fp64, CPU), used to compare against
the fixture recorded from the reference's own Python (tests/golden/modules_ref_python.npz).
Order of the pointwise stage as in picasso/mesh/layers.py:114-119,169-174: matmul -> + bias ->
ReLU -> BatchNorm1d(eps=1e-3) in training mode (biased batch variance)."""
import torch

from oracle import mesh_oracle as mo


def tail(x, bias, bn_weight, bn_bias, eps=1e-3):
    x = torch.relu(x + bias)
    mean, var = x.mean(0), x.var(0, unbiased=False)
    return (x - mean) / torch.sqrt(var + eps) * bn_weight + bn_bias


def v2v_forward(x, params, face, nf_count, vt_map, coeff, cfg):
    """params: dict name -> fp64 leaf tensor with the reference's state_dict names."""
    cin, mid, cout, L, m1, m2 = cfg
    sh_eye = mo.sph_harm_coeff(L, torch.eye(3)).double()
    spatial = (sh_eye @ params["V2F_conv3d.spatial_weights"]).reshape(3, cin, m1)
    y = mo.vertex2facet(x, spatial, face) @ params["V2F_conv3d.depth_weights"]
    y = tail(y, params["V2F_conv3d.biases"], params["V2F_conv3d.BatchNorm.weight"], params["V2F_conv3d.BatchNorm.bias"])
    z = mo.facet2vertex(y, params["F2V_conv3d.spatial_weights"], coeff, face, nf_count, vt_map)
    z = z @ params["F2V_conv3d.depth_weights"]
    return tail(z, params["F2V_conv3d.biases"], params["F2V_conv3d.BatchNorm.weight"], params["F2V_conv3d.BatchNorm.bias"])


def f2f_forward(tex, params, bary, counts):
    cum = torch.cumsum(counts, 0, dtype=torch.int32)
    z = mo.facet2facet(tex, params["weights"], bary, cum)
    return tail(z, params["biases"], params["BatchNorm.weight"], params["BatchNorm.bias"])


def load_fixture(name="modules_ref_python.npz"):
    import os
    import numpy as np
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", name)
    z = np.load(path)
    return {k: z[k] for k in z.files}


def group(fx, prefix):
    """{'name': tensor} for the fixture keys that start with prefix + '/'."""
    return {k[len(prefix) + 1:]: torch.from_numpy(v) for k, v in fx.items() if k.startswith(prefix + "/")}
