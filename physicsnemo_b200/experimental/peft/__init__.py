from .lora import (ApplyResult, LoRAConfig, LoRALayer, LoRALinear, apply_lora, compute_base_fingerprint, is_lora_layer, load_adapter,
                   merge_lora, print_trainable_parameters, register_lora_wrapper, resolve_targets, save_adapter, set_adapter_enabled,
                   split_params_for_optimizer, wrappable_types)

__all__ = ["ApplyResult", "LoRAConfig", "LoRALayer", "LoRALinear", "apply_lora", "compute_base_fingerprint", "is_lora_layer", "load_adapter",
           "merge_lora", "print_trainable_parameters", "register_lora_wrapper", "resolve_targets", "save_adapter", "set_adapter_enabled",
           "split_params_for_optimizer", "wrappable_types"]
