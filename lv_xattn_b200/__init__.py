"""B200-native LV-XAttn: sequence-parallel cross-attention behind the reference's `lv_xattn` interface.

Exports what reference lv_xattn/__init__.py:1-2 exports, plus the autograd wrappers its drivers build.
All compute runs in liblvx.so (sm_100a CUDA, C ABI in include/lvx.h); there is no CPU or Triton path.
"""
from .async_communication import (  # noqa: F401
    P2PTimeoutError,
    destroy_sequence_parallel,
    get_sequence_parallel_group,
    get_sequence_parallel_rank,
    get_sequence_parallel_size,
    initialize_distributed,
    reset_global_memory_buffer,
)
from .attn import (  # noqa: F401
    LVXAttnFunc,
    LVXAttnRecomputeFunc,
    RingAttnRecomputeFunc,
    _attn_backward,
    _attn_forward,
    attention,
    create_attention_class,
)
from .hf_patch import (  # noqa: F401,E402
    clear_global_cross_attention_states,
    get_global_cross_attention_states,
    install_hooks,
    patch_cross_attention_forward,
    patch_self_attention_forward,
    set_global_cross_attention_states,
    uninstall_hooks,
)
from .host_io import HostStreamedAttention  # noqa: F401,E402
from .peer_memory import check_device_status  # noqa: F401,E402
