"""B200-native packed-KV path behind the InQuant Python interface.

Module and symbol names follow the reference package (``inquant.codec``,
``inquant.value_codec``, ``inquant.cache``, ``inquant.triton_selection``,
``inquant.triton_attention``, ``inquant.qwen_fused``); every numeric operation runs in
hand-written sm_100a CUDA reached through the C ABI of ``libinquant_b200.so``.  There is
no Triton import, no alternative backend and no CPU fallback: CPU tensors are rejected.
"""

__version__ = "0.1.0"
