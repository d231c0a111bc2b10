"""Hot ops. On CUDA bf16 tensors each function runs a hand-written sm_100a kernel from
``libvmoe_b200.so``; on other tensors it runs the PyTorch restatement of the same contract,
which is also the oracle the kernels are tested against."""
from vmoe_b200.ops.functional import (attention, attention_packed, expert_mlp, layer_norm, layer_norm_fork, linear, use_cuda_kernels,
                                      cuda_kernels_enabled)
