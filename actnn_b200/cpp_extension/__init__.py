"""Python faces of the native library, one module per extension of the reference:
``minimax``, ``quantization``, ``calc_precision`` and ``backward_func``
(reference: actnn/setup.py:5-22).  Each function validates its tensors the way the
reference's TORCH_CHECK macros do (actnn/actnn/cpp_extension/ext_common.h:2-27, plus
bfloat16), allocates the outputs and forwards raw pointers to ``libactnn_b200.so``."""
