"""Paged (vLLM-extension) layout of the packed-KV path on B200: byte layout, direct page
sealing and paged decode with the interfaces of the reference's ``inquant_vllm`` package.
``backend`` holds the request state machine of the reference's attention backend; the vLLM
platform / worker plugin of the reference is engine integration and is not part of this build."""
