"""Linear BVH over the component means of each mixture (gmc_lbvh_build of libgmc_b200.so)."""
import torch

from . import _native


def build(mixture: torch.Tensor):
    """mixture [B, L, G, 7|13] (CUDA, fp32) -> (sorted_keys int64 [B, L, G], nodes int16 [B, L, 2G-1, 4]).

    key = (30-bit Morton code of the mean in the mixture's own bounding box) << 16 | component id; nodes are
    {parent, left, right, object} with internal nodes first (root 0) and leaves in sorted-key order."""
    if mixture.dim() != 4 or mixture.shape[-1] not in (7, 13):
        raise RuntimeError("mixture must be [batch, layers, components, 7 or 13]")
    mixture = mixture.contiguous()
    _native.require_cuda_f32(mixture, "mixture")
    b, l, g, v = mixture.shape
    keys = torch.empty((b, l, g), dtype=torch.int64, device=mixture.device)
    nodes = torch.empty((b, l, 2 * g - 1, 4), dtype=torch.int16, device=mixture.device)
    with torch.cuda.device_of(mixture):
        _native.check(_native.lib.gmc_lbvh_build(_native.ptr(mixture), b * l, g, 2 if v == 7 else 3,
                                                 _native.ptr(keys), _native.ptr(nodes), _native.stream_of(mixture)),
                      "lbvh build")
    return keys, nodes
