"""B200-native calibrate-and-quantize path behind the llm-compressor API.

    from llm_compressor_b200 import oneshot, GPTQModifier, QuantizationModifier

Compute runs in ``libb200q.so`` (hand-written sm_100a CUDA, C ABI in ``include/b200q.h``);
this package is the host-side mirror of the reference's interfaces for that path.
"""
from .quant_args import QuantizationArgs, QuantizationScheme, preset_name_to_scheme  # noqa: F401
from .observers import Observer  # noqa: F401
from .gptq import (accumulate_hessian, make_empty_hessian, quantize_weight,  # noqa: F401
                   factor_hessian, finalize_hessian, accumulate_hessian_lower)
from .modifiers import GPTQModifier, QuantizationModifier, match_named_modules  # noqa: F401
from .awq import AWQMapping, AWQModifier  # noqa: F401
from .oneshot import oneshot, save_compressed_model  # noqa: F401
from .compressors import compress_state_dict, infer_module_format  # noqa: F401
from .model_free import model_free_ptq  # noqa: F401
