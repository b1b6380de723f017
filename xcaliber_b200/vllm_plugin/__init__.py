"""vLLM plugin slot of the B200 fused MoE operator (the reference's counterpart is the package
xFused-XXXX-Kernels/xMoE/xW4A16/sm75/xR64/vllm/xcaliber_int4_vllm). Activate with the entry point
group `vllm.general_plugins` -> `xcaliber_b200.vllm_plugin.plugin:register` and VLLM_PLUGINS."""
