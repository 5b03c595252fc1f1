"""``spconv.pytorch.cppcore`` by name: upstream converts torch tensors to its own
tensor-view objects there.  This package passes raw device pointers to its C
library instead, so only the stream helper has a meaning here."""

import torch


def get_current_stream() -> int:
    """Handle (``cudaStream_t`` as an integer) of the current CUDA stream, 0 without CUDA."""
    return torch.cuda.current_stream().cuda_stream if torch.cuda.is_available() else 0


def torch_tensor_to_tv(*args, **kwargs):
    raise NotImplementedError("there are no tensor-view objects in spconv_triton_b200; pass torch tensors")
