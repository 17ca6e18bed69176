"""Bindings of the sm_100a kernels into the hosts of the reference: its own package (``binding``) and the vLLM plugin
slot hooks selected by ``STATEQUANT_VLLM`` (``vllm_plugin``)."""
