from .lora import (AdapterConfig, LoRA, LoHa, LoKr, DoRA, IA3, GLoRA, LoConConv2d,  # noqa: F401
                   AdaptedConv2d, inject_adapters, adapter_parameters, adapter_state_dict,
                   load_adapter_state_dict, load_adapters_into, merge_adapters)
