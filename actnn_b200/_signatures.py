"""Argument types of every status-returning entry point of ``libactnn_b200.so``, exactly as
declared in ``include/actnn_b200.h``.  One letter per argument:

    P  pointer (device or host) or ``None``      I  int           L  int64_t
    U  uint64_t                                  F  float         D  double

Kept free of imports so that the build script can read it without loading torch."""

SIGNATURES = {
    "actnn_minimax": ['P', 'P', 'P', 'L', 'L', 'I', 'P'],
    "actnn_bits_prefix": ['P', 'L', 'L', 'L', 'P', 'P'],
    "actnn_pack_mixed": ['P', 'P', 'P', 'P', 'P', 'P', 'P', 'P', 'L', 'L', 'L', 'I', 'I', 'I', 'P', 'U', 'U', 'P'],
    "actnn_unpack_mixed": ['P', 'P', 'P', 'P', 'P', 'P', 'L', 'L', 'L', 'I', 'I', 'P'],
    "actnn_pack_single": ['P', 'P', 'P', 'I', 'P', 'P', 'P', 'L', 'L', 'L', 'I', 'I', 'I', 'P', 'U', 'U', 'P'],
    "actnn_unpack_single": ['P', 'I', 'P', 'P', 'P', 'L', 'L', 'L', 'I', 'I', 'P'],
    "actnn_compress_single": ['P', 'I', 'P', 'P', 'P', 'P', 'L', 'L', 'L', 'I', 'I', 'I', 'P', 'U', 'U', 'P'],
    "actnn_compress_mixed": ['P', 'P', 'P', 'P', 'P', 'P', 'P', 'P', 'L', 'L', 'L', 'L', 'I', 'I', 'F', 'F', 'P', 'I', 'D', 'I', 'P',
                             'U', 'U', 'P'],
    "actnn_compress_mixed_static": ['P', 'P', 'P', 'P', 'P', 'P', 'P', 'L', 'L', 'L', 'I', 'I', 'F', 'F', 'P', 'I', 'D', 'I', 'P', 'U',
                                    'U', 'P'],
    "actnn_compress_mixed_prestat": ['P', 'P', 'P', 'P', 'P', 'P', 'P', 'P', 'P', 'P', 'L', 'L', 'L', 'I', 'I', 'F', 'F', 'P', 'I', 'D', 'I',
                                     'P', 'U', 'U', 'P'],
    "actnn_compress_mixed_prestat_kept": ['P'] * 10 + ['L', 'L', 'L', 'I', 'I', 'F', 'F', 'P', 'I', 'D', 'I', 'P', 'U', 'U',
                                          'P'],
    "actnn_batch_norm_stats_minimax": ['P'] * 9 + ['L', 'L', 'L', 'D', 'D', 'I', 'P', 'L', 'P'],
    "actnn_range_sqr": ['P', 'P', 'L', 'L', 'I', 'F', 'F', 'P', 'P', 'P'],
    "actnn_sample_sumsq": ['P', 'P', 'L', 'L', 'I', 'P'],
    "actnn_calc_precision": ['P', 'P', 'L', 'I', 'D', 'P', 'P', 'L', 'L', 'P', 'L', 'P'],
    "actnn_relu_forward": ['P', 'P', 'P', 'L', 'I', 'P'],
    "actnn_relu_forward_minimax": ['P', 'P', 'P', 'P', 'P', 'L', 'I', 'P'],
    "actnn_relu_backward": ['P', 'P', 'P', 'L', 'I', 'P'],
    "actnn_dropout_forward": ['P', 'P', 'P', 'L', 'F', 'I', 'P', 'U', 'U', 'P'],
    "actnn_dropout_backward": ['P', 'P', 'P', 'L', 'F', 'I', 'P'],
    "actnn_dropout_uniform_fill": ['P', 'L', 'U', 'U', 'P'],
    "actnn_max_pool2d_forward": ['P', 'P', 'P', 'L', 'L', 'L', 'L'] + ['I'] * 9 + ['P'],
    "actnn_max_pool2d_backward": ['P', 'P', 'P', 'L', 'L', 'L', 'L'] + ['I'] * 9 + ['P'],
    "actnn_noise_fill": ['P', 'L', 'I', 'U', 'U', 'P'],
    "actnn_bulk_wait_failures": ['P'],
    "actnn_bad_width_bundles": ['P'],
    "actnn_batch_norm_stats": ['P', 'P', 'P', 'L', 'L', 'L', 'D', 'I', 'P', 'L', 'P'],
    "actnn_batch_norm_elemt": ['P'] * 6 + ['L', 'L', 'L', 'I', 'P', 'L', 'P'],
    "actnn_batch_norm_backward_reduce": ['P'] * 8 + ['L', 'L', 'L', 'I', 'P', 'L', 'P'],
    "actnn_batch_norm_backward_elemt": ['P'] * 8 + ['L', 'P', 'L', 'L', 'L', 'I', 'P', 'L', 'P'],
    "actnn_batch_norm_forward": ['P'] * 8 + ['L', 'L', 'L', 'D', 'D', 'I', 'P', 'L', 'P'],
    "actnn_batch_norm_backward": ['P'] * 8 + ['L', 'L', 'L', 'I', 'P', 'L', 'P'],
}
