"""The reference's import statements work unchanged (actnn/actnn/ops.py:15-17,
mem_speed_benchmark/train.py:29-31,292) and name the same objects as ``actnn_b200``."""


def test_reference_import_statements_resolve_to_this_library():
    import actnn
    from actnn import config, QScheme, QModule                                   # noqa: F401
    from actnn import get_memory_usage, compute_tensor_bytes, exp_recorder       # noqa: F401
    from actnn.layers import QConv2d, QBatchNorm2d, QLinear                      # noqa: F401
    import actnn.cpp_extension.calc_precision as ext_calc_precision
    import actnn.cpp_extension.minimax as ext_minimax
    import actnn.cpp_extension.quantization as ext_quantization
    import actnn.cpp_extension.backward_func as ext_backward_func
    from actnn.ops import quantize_activation, dequantize_activation            # noqa: F401
    from actnn.qscheme import QScheme as QS2
    from actnn.conf import config as config2

    import actnn_b200
    assert actnn.config is actnn_b200.config is config is config2
    assert QScheme is actnn_b200.QScheme is QS2
    assert actnn.ops is actnn_b200.ops
    assert ext_quantization is actnn_b200.cpp_extension.quantization
    for mod, names in ((ext_minimax, ["minimax"]), (ext_calc_precision, ["calc_precision"]),
                       (ext_quantization, ["pack_mixed_precision", "unpack_mixed_precision", "pack_single_precision",
                                           "unpack_single_precision", "act_quantized_relu", "act_quantized_dropout",
                                           "act_quantized_max_pool2d"]),
                       (ext_backward_func, ["cudnn_convolution_backward", "cudnn_convolution_transpose_backward",
                                            "cudnn_batch_norm", "cudnn_batch_norm_backward", "native_batch_norm",
                                            "native_batch_norm_backward"])):
        for name in names:
            assert callable(getattr(mod, name)), name
    actnn.set_optimization_level("L3")
    assert actnn_b200.config.compress_activation and actnn_b200.config.activation_compression_bits[0] == 2
    actnn.set_optimization_level("L0")
