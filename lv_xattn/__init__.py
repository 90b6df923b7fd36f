"""Drop-in alias: `from lv_xattn import _attn_forward, _attn_backward, initialize_distributed,
reset_global_memory_buffer, get_sequence_parallel_group` resolves to the B200 implementation
(the names reference lv_xattn/__init__.py:1-2 exports)."""
from lv_xattn_b200 import *  # noqa: F401,F403
from lv_xattn_b200 import _attn_backward, _attn_forward  # noqa: F401
from lv_xattn_b200 import async_communication, attn  # noqa: F401
