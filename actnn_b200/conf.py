"""Global configuration and optimisation levels.

Same switches, defaults and level table as the reference (actnn/actnn/conf.py:5-68);
``actnn.config`` is one mutable, process-wide object there and so it is here."""
import ast
import os
import warnings


class QuantizationConfig:
    def __init__(self):
        # what gets compressed and how
        self.compress_activation = True
        self.activation_compression_bits = [2, 8, 8]     # average bits per layer "group"
        self.pergroup = True
        self.perlayer = True
        self.initial_bits = 8
        self.stochastic = True
        self.training = True
        self.group_size = 256
        self.use_gradient = False
        self.adaptive_conv_scheme = True
        self.relu_minmax = True        # QReLU also produces the group ranges of its output (not in the reference)
        self.adaptive_bn_scheme = True
        self.simulate = False
        self.enable_quantized_bn = True

        # memory management
        self.empty_cache_threshold = None
        self.pipeline_threshold = None
        self.cudnn_benchmark_conv2d = True
        self.swap = False
        self.swap_arena = True                 # pooled pinned buffers + copy streams for the swap (False: the reference's scheme)

        # debugging
        self.debug_memory_model = ast.literal_eval(os.environ.get("DEBUG_MEM", "False"))
        self.debug_speed = ast.literal_eval(os.environ.get("DEBUG_SPEED", "False"))
        self.debug_memory_op_forward = False
        self.debug_memory_op_backward = False
        self.debug_remove_bn = False
        self.debug_remove_relu = False


config = QuantizationConfig()


def _no_adaptive():
    config.adaptive_conv_scheme = config.adaptive_bn_scheme = False


def set_optimization_level(level: str) -> None:
    """L0 exact .. L5 2-bit + swap + defragmentation; ``swap`` = offload only."""
    if level == "L0":
        config.compress_activation = False
        _no_adaptive()
    elif level == "L1":                       # 4-bit conv inputs, exact batch norm
        config.activation_compression_bits = [4]
        _no_adaptive()
        config.enable_quantized_bn = False
    elif level == "L2":                       # 4-bit everywhere
        config.activation_compression_bits = [4]
        _no_adaptive()
    elif level == "L3":                       # 2-bit average, per-sample and per-layer adaptive
        pass
    elif level == "L3.1":                     # L3 + light system tweaks
        config.cudnn_benchmark_conv2d = False
        config.empty_cache_threshold = 0.2
        config.pipeline_threshold = 3 * 1024 ** 3
    elif level == "L4":                       # L3 + packed tensors swapped to pinned host memory
        config.swap = True
    elif level == "L5":                       # L4 + allocator defragmentation
        config.swap = True
        os.environ["PYTORCH_CACHE_THRESHOLD"] = "256000000"
        warnings.warn("The defragmentation of L5 relies on a patched PyTorch allocator "
                      "(https://github.com/merrymercy/pytorch/tree/actnn_exp); without it L5 behaves like L4.")
    elif level == "swap":
        config.swap = True
        config.compress_activation = False
    else:
        raise ValueError("Invalid level: " + level)
