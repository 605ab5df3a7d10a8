"""Quantization scheme for batch-norm inputs: sensitivity = range only, bits follow the
preceding conv / linear layer (mirror of actnn/actnn/qbnscheme.py:9-60)."""
from .conf import config
from .cpp_extension import calc_precision as ext_calc_precision
from .cpp_extension import quantization as ext_quantization
from .qscheme import QScheme, group_minimax, to_groups, total_bits_after_greedy


class QBNScheme(QScheme):
    layers = []

    def __init__(self, group=0):
        self.initial_bits = config.initial_bits
        self.bits = config.activation_compression_bits[group]
        QBNScheme.layers.append(self)
        self.prev_linear = QScheme.layers[-1] if len(QScheme.layers) > 0 else None

    def compute_quantization_bits(self, input):
        self.prev_linear = QScheme.prev_layer
        N, D = input.shape[0], input.shape[1]
        num_pixels = (input.numel() // N) // D
        groups, mn, mx = group_minimax(input)
        G = groups.shape[1]
        C = ext_calc_precision.sensitivity(mn, mx, N, config.group_size / num_pixels)
        target = int(self.bits * N)
        b, offsets = ext_calc_precision.allocate_bits(C, self.initial_bits, target, None, G,
                                                      config.group_size, with_offsets=True)
        b.word_offsets = offsets
        b.total_bits = total_bits_after_greedy(N, self.initial_bits, target)
        return groups, b, mn, mx

    def compress(self, input, stat_dtype, minmax=None):
        """One-call variant of ``compute_quantization_bits`` + pack (see ``QScheme.compress``).
        ``minmax``: group extrema already computed together with the batch-norm statistics."""
        if not config.pergroup:
            return None
        self.prev_linear = QScheme.prev_layer
        N, D = input.shape[0], input.shape[1]
        num_pixels = (input.numel() // N) // D
        q_input, b, q_scale, q_min, _ = ext_quantization.compress_mixed_precision(
            to_groups(input), int(self.bits * N), int(self.initial_bits), config.group_size / num_pixels,
            1.0, None, config.stochastic, stat_dtype=stat_dtype, minmax=minmax)
        return q_input, b, q_scale, q_min

    @staticmethod
    def allocate_perlayer():
        for layer in QBNScheme.layers:
            layer.bits = layer.prev_linear.bits if layer.prev_linear is not None else 8
