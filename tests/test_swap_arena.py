"""The host swap arena: pool bookkeeping on the CPU, copies and ordering on a GPU."""
import pytest
import torch


def test_stack_reuses_memory_across_steps_whatever_the_block_sizes():
    from actnn_b200.swap_arena import PinnedStack
    made = []

    def alloc(n):
        made.append(n)
        return torch.zeros(n, dtype=torch.uint8)

    stack = PinnedStack(alloc, slab_bytes=10000)
    # step 1: three blocks, freed newest first
    b1, t1 = stack.push(3000)
    b2, t2 = stack.push(100)
    b3, t3 = stack.push(4000)
    assert b1.numel() == 3000 and b2.numel() == 100 and b3.numel() == 4000 and made == [10000]
    assert b1.data_ptr() % 512 == b2.data_ptr() % 512 == b3.data_ptr() % 512        # 512-byte spacing
    assert stack.live_bytes == 3072 + 512 + 4096
    for t in (t3, t2, t1):
        stack.pop(t)
    assert stack.live_bytes == 0
    # step 2: different sizes, same total: no new slab, memory starts at the same place
    c1, u1 = stack.push(5000)
    c2, u2 = stack.push(2100)
    assert made == [10000] and c1.data_ptr() == b1.data_ptr()
    # blocks of one step never overlap
    c1.fill_(1)
    c2.fill_(2)
    assert int(c1.sum()) == 5000 and int(c2.sum()) == 4200
    # a block that does not fit the slab goes to a second one; an oversized block gets its own
    c3, u3 = stack.push(6000)
    assert made == [10000, 10000]
    c4, u4 = stack.push(25000)
    assert made == [10000, 10000, 25088] and c4.numel() == 25000
    assert stack.allocated_bytes == 45088
    # out-of-order frees only delay the fall-back
    stack.pop(u2)
    stack.pop(u1)
    assert stack.live_bytes == 6144 + 25088
    stack.pop(u4)
    stack.pop(u4)                                   # popping twice is harmless
    d, v = stack.push(100)                          # lands right after c3 in the second slab
    assert made == [10000, 10000, 25088] and d.data_ptr() == c3.data_ptr() + 6144
    stack.pop(v)
    stack.pop(u3)
    assert stack.live_bytes == 0 and stack.peak_live_bytes >= 6144 + 25088
    e, _ = stack.push(64)
    assert e.data_ptr() == b1.data_ptr()


@pytest.fixture()
def actnn(cuda_device):
    import actnn_b200
    from actnn_b200.conf import QuantizationConfig
    from actnn_b200 import swap_arena
    fresh = QuantizationConfig()
    actnn_b200.config.__dict__.update(fresh.__dict__)
    yield actnn_b200
    actnn_b200.config.__dict__.update(fresh.__dict__)
    swap_arena.reset_arenas()


@pytest.mark.gpu
def test_round_trip_in_stack_order_and_out_of_order(actnn, cuda_device):
    from actnn_b200.utils import swap_to_cpu, swap_to_gpu
    from actnn_b200.swap_arena import SwappedTensor, arena_for
    g = torch.Generator(device="cuda").manual_seed(0)
    originals, handles = [], []
    for i in range(24):
        shape = (3 + i, 1000 * (i % 5 + 1) + 7)
        t = torch.randint(-2 ** 31, 2 ** 31 - 1, shape, dtype=torch.int32, device="cuda", generator=g)
        if i % 3 == 0:
            t = t.to(torch.int8)
        t.word_offsets = ("offsets", i)
        originals.append(t.clone())
        handles.append(swap_to_cpu(t))
        del t
        torch.empty(1 << 22, device="cuda").fill_(1.0)      # churn the allocator behind the copies
    assert all(isinstance(h, SwappedTensor) for h in handles)
    order = list(range(23, 11, -1)) + [2, 9, 0, 5, 11, 1, 3, 4, 6, 7, 8, 10]
    for i in order:
        back = swap_to_gpu(handles[i])
        assert back.is_cuda and back.dtype == originals[i].dtype and torch.equal(back, originals[i])
        assert back.word_offsets == ("offsets", i)
    with pytest.raises(RuntimeError):
        swap_to_gpu(handles[0])
    arena = arena_for(cuda_device)
    first = arena.pool.allocated_bytes
    assert arena.pool.live_bytes == 0
    # a second "step" of the same sizes pins no new memory
    handles = [swap_to_cpu(o) for o in originals]
    assert arena.pool.allocated_bytes == first
    for h, o in zip(reversed(handles), reversed(originals)):
        assert torch.equal(swap_to_gpu(h), o)
    # handles that are never fetched give their buffers back
    handles = [swap_to_cpu(o) for o in originals]
    del handles, h
    torch.cuda.synchronize()
    again = [swap_to_cpu(o) for o in originals]
    assert arena.pool.allocated_bytes == first
    for h, o in zip(again, originals):
        assert torch.equal(swap_to_gpu(h), o)


@pytest.mark.gpu
@pytest.mark.parametrize("level", ["L4", "swap"])
def test_swapped_training_step_equals_the_unswapped_one(actnn, level):
    """Same seed, same noise: gradients with the activations parked in host memory equal the
    gradients with them kept on the device, for the arena and for the reference's scheme."""
    import torch.nn as nn

    def grads(swap, arena):
        actnn.config.__dict__.update(type(actnn.config)().__dict__)
        actnn.QScheme.layers.clear()
        actnn.QBNScheme.layers.clear()
        actnn.set_optimization_level("L3" if level == "L4" else "L0")
        actnn.config.swap = swap
        actnn.config.swap_arena = arena
        if level == "swap":
            actnn.config.compress_activation = False
        torch.manual_seed(0)
        net = nn.Sequential(nn.Conv2d(3, 16, 3, padding=1), nn.BatchNorm2d(16), nn.ReLU(),
                            nn.Conv2d(16, 32, 3, padding=1), nn.BatchNorm2d(32), nn.ReLU(),
                            nn.AdaptiveAvgPool2d(1), nn.Flatten(), nn.Linear(32, 10)).cuda()
        q = actnn.QModule(net).train()
        x = torch.randn(32, 3, 32, 32, device="cuda")
        y = torch.randint(0, 10, (32,), device="cuda")
        out = []
        for _ in range(2):                                   # the second step has real gradient scales
            q.zero_grad(set_to_none=True)
            torch.manual_seed(1)
            nn.functional.cross_entropy(q(x), y).backward()
            out = [p.grad.clone() for p in q.parameters()]
        return out

    base = grads(False, True)
    for arena in (True, False):
        got = grads(True, arena)
        assert len(got) == len(base)
        for a, b in zip(got, base):                          # cuDNN's weight gradients are not bit-reproducible
            assert torch.allclose(a, b, rtol=1e-4, atol=1e-6 * float(b.abs().max()) + 1e-9)
