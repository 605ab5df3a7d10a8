"""Per-layer quantization scheme for conv / linear inputs: per-sample sensitivities and the
greedy per-sample bit allocation, entirely on the device.

Behavioural mirror of actnn/actnn/qscheme.py:9-147.  The reference computes the
sensitivities with half a dozen small torch kernels, copies them to the host, runs a CPU
priority queue and copies the bits back (three host synchronisations per layer per
step).  Here the chain is minimax -> sensitivity -> allocate_bits, three kernel launches
with no host round trip; the only host read left is the once-per-step per-layer
re-allocation."""
import torch

from .conf import config
from .cpp_extension import calc_precision as ext_calc_precision
from .cpp_extension import minimax as ext_minimax
from .cpp_extension import quantization as ext_quantization


def to_groups(input: torch.Tensor) -> torch.Tensor:
    """Flatten to ``[N, G, group_size]``, zero-padding the tail of every sample (qscheme.py:61-71)."""
    N = input.shape[0]
    gs = config.group_size
    flat = input.view(N, -1)
    num_features = flat.shape[1]
    if num_features % gs != 0:
        pad = (num_features // gs + 1) * gs - num_features
        flat = torch.cat([flat, torch.zeros([N, pad], dtype=input.dtype, device=input.device)], 1)
    return flat.view(N, -1, gs)


def group_minimax(input: torch.Tensor):
    """``(groups [N,G,gs], mn[N,G,1], mx[N,G,1])`` of an activation."""
    N = input.shape[0]
    gs = config.group_size
    groups = to_groups(input).view(-1, gs)
    mn, mx = ext_minimax.minimax(groups)
    if not config.pergroup:                       # one range for the whole tensor
        mn = torch.ones_like(mn) * mn.min()
        mx = torch.ones_like(mx) * mx.max()
    return groups.view(N, -1, gs), mn.view(N, -1, 1), mx.view(N, -1, 1)


def total_bits_after_greedy(n: int, initial_bits: int, target: int) -> int:
    """sum(bits) the greedy ends with (unit weights): it removes one bit at a time from
    ``initial_bits * n`` until the sum is <= target and cannot go below one bit each."""
    return min(initial_bits * n, max(int(target), n))


class QScheme(object):
    num_samples = 1
    num_layers = 0
    batch = None
    update_scale = True
    layers = []
    prev_layer = None

    def __init__(self, layer, group=0, num_locations=1, depthwise_groups=1):
        self.initial_bits = config.initial_bits
        self.bits = config.activation_compression_bits[group]
        if config.use_gradient:
            assert QScheme.num_samples > 1
            self.scales = torch.zeros(QScheme.num_samples)
        else:
            self.scales = torch.tensor([0.0])
        QScheme.layers.append(self)
        self.C = None
        self.dim = None
        self.num_locations = num_locations            # kernel taps
        self.depthwise_groups = depthwise_groups
        self.layer = layer
        self.group = group
        self.name = "layer_{}".format(QScheme.num_layers)
        QScheme.num_layers += 1

    # ------------------------------------------------------------- gradient scale
    def get_scale(self):
        if config.use_gradient:
            assert QScheme.batch is not None
            scale = self.scales[QScheme.batch].clone()
            avg_scale = scale.mean()
            scale[scale == 0] = avg_scale + 1e-9
            return scale
        return self.scales

    def set_scale(self, grad):
        if not QScheme.update_scale:
            return
        sq = ext_calc_precision.sample_sumsq(grad)
        if config.use_gradient:
            assert QScheme.batch is not None
            self.scales[QScheme.batch] = self.scales[QScheme.batch] * 0.5 + sq.cpu() * 0.5
        else:
            self.scales = sq.mean()

    # ------------------------------------------------------------- per-sample bits
    def _sensitivity(self, mn, mx, N, range_factor, device):
        coeff = self.num_locations / 4 / self.depthwise_groups
        grad = self.get_scale()
        if grad.numel() == 1:
            if not grad.is_cuda or grad.dtype != torch.float32:
                grad = grad.to(device=device, dtype=torch.float32)
                if not config.use_gradient:
                    self.scales = grad                 # keep it on the device from now on
            return ext_calc_precision.sensitivity(mn, mx, N, range_factor, coeff, grad.reshape(1))
        C = ext_calc_precision.sensitivity(mn, mx, N, range_factor, coeff)
        return C * grad.to(device=device, dtype=torch.float32)

    def compute_quantization_bits(self, input):
        QScheme.prev_layer = self
        N, D = input.shape[0], input.shape[1]
        num_pixels = (input.numel() // N) // D
        groups, mn, mx = group_minimax(input)
        G = groups.shape[1]
        C = self._sensitivity(mn, mx, N, config.group_size / num_pixels, input.device)
        target = int(self.bits * N)
        b, offsets = ext_calc_precision.allocate_bits(C, self.initial_bits, target, None, G,
                                                      config.group_size, with_offsets=True)
        b.word_offsets = offsets
        b.total_bits = total_bits_after_greedy(N, self.initial_bits, target)
        self.C = C
        self.dim = input.numel() // N
        self.b = b
        return groups, b, mn, mx

    def compress(self, input, stat_dtype, minmax=None):
        """``compute_quantization_bits`` + mixed-precision pack as ONE native call (three kernel
        launches, no host synchronisation).  Returns ``(q_input, q_bits, q_scale, q_min)``, or
        ``None`` when a configuration needs the step-by-step path.  ``minmax=(mn, mx)``: the
        per-group extrema when the producer of ``input`` already has them (then the activation is
        read once, not twice); only used when every sample is whole groups of 256."""
        grad = self.get_scale()
        if not config.pergroup or grad.numel() != 1:
            return None
        QScheme.prev_layer = self
        N, D = input.shape[0], input.shape[1]
        num_pixels = (input.numel() // N) // D
        if not grad.is_cuda or grad.dtype != torch.float32:
            grad = grad.to(device=input.device, dtype=torch.float32)
            self.scales = grad
        if minmax is not None and (config.group_size != 256 or (input.numel() // N) % 256 != 0):
            minmax = None                                      # padded groups: not the producer's
        q_input, b, q_scale, q_min, C = ext_quantization.compress_mixed_precision(
            to_groups(input), int(self.bits * N), int(self.initial_bits), config.group_size / num_pixels,
            self.num_locations / 4 / self.depthwise_groups, grad.reshape(1), config.stochastic,
            stat_dtype=stat_dtype, minmax=minmax)
        self.C = C
        self.dim = input.numel() // N
        self.b = b
        return q_input, b, q_scale, q_min

    # ------------------------------------------------------------- per-layer bits
    @staticmethod
    def allocate_perlayer():
        for g, group_bits in enumerate(config.activation_compression_bits):
            layers = [layer for layer in QScheme.layers if layer.group == g and layer.C is not None]
            L = len(layers)
            if L == 0:
                continue
            device = layers[0].C.device
            if group_bits == config.initial_bits:
                # one width per layer: weight = features per sample
                C = torch.stack([layer.C.sum() for layer in layers]).to(torch.float32)
                w = torch.tensor([layer.dim for layer in layers], dtype=torch.int32, device=device)
                total = float(sum(layer.dim for layer in layers) * group_bits)
                b, _ = ext_calc_precision.allocate_bits(C.contiguous(), 8, total, w)
                b = b.cpu()
                for i, layer in enumerate(layers):
                    layer.bits = layer.initial_bits = b[i]
            else:
                # joint allocation over layers x samples, then the per-layer average
                N = layers[0].C.shape[0]
                C = torch.cat([layer.C for layer in layers], 0).contiguous()
                w = torch.tensor([layer.dim for layer in layers], dtype=torch.int32,
                                 device=device).repeat_interleave(N).contiguous()
                total = float(sum(layer.dim for layer in layers) * N * group_bits)
                b, _ = ext_calc_precision.allocate_bits(C, config.initial_bits, total, w)
                # the one host read per step.  Integer sums are exact on any device; the division
                # is done on the host in float32 like the reference's ``bs.float().mean()``
                means = b.view(L, N).sum(dim=1).cpu().float() / N
                for i, layer in enumerate(layers):
                    layer.bits = means[i]

    def if_allocate_perlayer(self):
        """Called at the end of every layer's backward; re-allocates the per-layer widths when
        backward has reached the first trainable layer (qscheme.py:130-147 of the reference).
        The cheap test (is this that layer?) comes first: the scans below are O(layers)."""
        if not config.perlayer or not (config.compress_activation and config.training):
            return
        first_layer = None
        for layer in QScheme.layers:
            if layer.layer.weight.requires_grad:
                first_layer = layer
                break
        # backward reaches the first trainable layer last: re-allocate there
        if self is not first_layer:
            return
        for layer in QScheme.layers:
            if layer.C is None:
                return
        from .qbnscheme import QBNScheme
        QScheme.allocate_perlayer()
        QBNScheme.allocate_perlayer()
