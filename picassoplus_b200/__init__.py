"""picassoplus_b200: the mesh-convolution path of PicassoPlus (vertex->facet, facet->facet,
facet->vertex, forward and backward, spherical-harmonic filter bases) as CUDA kernels for
NVIDIA B200 (sm_100a) behind the reference's operator API.

    from picassoplus_b200.mesh.pi_modules import conv3d      # v2f_Function, f2f_Function, f2v_Function
    from picassoplus_b200.mesh.layers import V2VConv3d        # nn.Module wrappers
"""
__version__ = "0.1.0"
