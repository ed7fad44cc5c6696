"""B200-native bidirectional attention (forward + backward, dense and packed varlen) for
nanobrain's 3D ViT-B masked autoencoder: hand-written sm_100a kernels behind a C ABI, wrapped
as ``torch.library`` custom ops with the ``F.scaled_dot_product_attention`` signature."""

from .host_pipeline import HostPipeline
from .ops import check_status, sdpa, sdpa_varlen, selftest_mma

__all__ = ["sdpa", "sdpa_varlen", "check_status", "selftest_mma", "HostPipeline"]
