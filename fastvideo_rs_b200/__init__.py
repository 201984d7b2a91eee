"""B200-native (sm_100a) implementation of the Wan DiT self-attention hot path of
zaitrarrio/fastvideo-rs, behind that project's `rt::sdpa::sdpa` entry and `rt::sdpa_rule` chooser.

The compute lives in libfvsdpa.so (CUDA kernels + C ABI, see include/fv_sdpa.h); the modules here
are the host-side mirror of the reference interface over torch tensors:

    sdpa       Plan, BlockCausal, sdpa(), dense_fwd()
    sdpa_rule  Probe, FlashKernel, dense_route(), mma_kernel(), ...
    wan        rope tables, q/k RMSNorm + RoPE prologue, WanSelfAttention
    sp         shard_ranges and the sequence-parallel attention
    vsa        TilePlan and video sparse attention
"""
from ._lib import Declined, FvError  # noqa: F401
