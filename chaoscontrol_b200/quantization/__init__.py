from .gptq import (GPTQQuantizer, ar_self_generated_calibration, collect_hessians,
                   dequantize_state_dict, quantize_int6_gptq, quantize_int6_percentile)
from .packaging import pack_int6_lzma, unpack_int6_lzma

__all__ = ["GPTQQuantizer", "ar_self_generated_calibration", "collect_hessians", "dequantize_state_dict",
           "quantize_int6_gptq", "quantize_int6_percentile", "pack_int6_lzma", "unpack_int6_lzma"]
