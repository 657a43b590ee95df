"""Linear BVH over the component means of each mixture (gmc_lbvh_build of libgmc_b200.so)."""
import torch

from . import _native


#: key layouts of the reference's lbvh::Config::MortonCodeAlgorithm (src/gmc/cpp/extensions/lbvh/Config.h)
OLD, COV1_12P36PC16I, COV2_54PC10I, COV3_27P27C10I, COV4_27C27P10I = range(5)


def build(mixture: torch.Tensor, morton_code_algorithm: int = OLD, make_aabbs: bool = False, aabb_threshold: float = 0.001):
    """mixture [B, L, G, 7|13] (CUDA, fp32) -> (sorted_keys int64 [B, L, G], nodes int16 [B, L, 2G-1, 4])
    and, with make_aabbs, aabbs fp32 [B, L, 2G-1, 8] = {upper.xyz, 0, lower.xyz, 0} as a third result.

    key = (30-bit Morton code of the mean in the mixture's own bounding box) << 16 | component id (or one of the
    covariance-aware layouts); nodes are {parent, left, right, object} with internal nodes first (root 0) and leaves in
    sorted-key order. make_aabbs expects INVERSE covariances in the matrix slot and works with layouts 0 and 1
    (the options of lbvh::Config; lbvh/bvh.cu:164-231, 241-299)."""
    if mixture.dim() != 4 or mixture.shape[-1] not in (7, 13):
        raise RuntimeError("mixture must be [batch, layers, components, 7 or 13]")
    mixture = mixture.contiguous()
    _native.require_cuda_f32(mixture, "mixture")
    b, l, g, v = mixture.shape
    keys = torch.empty((b, l, g), dtype=torch.int64, device=mixture.device)
    nodes = torch.empty((b, l, 2 * g - 1, 4), dtype=torch.int16, device=mixture.device)
    aabbs = torch.empty((b, l, 2 * g - 1, 8), dtype=torch.float32, device=mixture.device) if make_aabbs else None
    with torch.cuda.device_of(mixture):
        _native.check(_native.lib.gmc_lbvh_build_ex(_native.ptr(mixture), b * l, g, 2 if v == 7 else 3,
                                                    int(morton_code_algorithm), int(bool(make_aabbs)), float(aabb_threshold),
                                                    _native.ptr(keys), _native.ptr(nodes),
                                                    _native.ptr(aabbs) if make_aabbs else None,
                                                    _native.stream_of(mixture)),
                      "lbvh build")
    return (keys, nodes, aabbs) if make_aabbs else (keys, nodes)
