"""GPU tests of the tensor-parallel MLP on two GPUs (skipped where fewer are visible): the library's
sum through peer memory against the rank-order fp32 sum computed from gathered partials (bit for
bit, on both ranks, across many calls and sizes), the sharded MLP against the unsharded one, and a
bounded wait that runs out because the peer makes its call late (made on the host: no kernel faults
or hangs; the late rank then completes the same call normally).

Each case runs as two child processes, one per GPU, over NCCL on 127.0.0.1 with NVLS off."""

import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _child(rank, world, port, case, results):
    import time

    import torch.distributed as dist

    from metile_b200 import _lib, synth
    from metile_b200 import backends as B
    from metile_b200 import tp

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    device = torch.device(f"cuda:{rank}")
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        if case in ("sum", "sum_two_shot"):
            hidden = 5120
            exchange = tp.PeerAllReduce(device, rank, world, 128 * hidden,
                                        mode="two_shot" if case == "sum_two_shot" else "auto")
            checked = 0
            for call, rows in enumerate([1, 128, 16, 1, 1, 64, 128, 2] * 4):
                partial = synth.activations(1000 + 10 * call + rank, rows, hidden, device)
                gathered = [torch.empty_like(partial) for _ in range(world)]
                dist.all_gather(gathered, partial)
                expected = gathered[0].float()
                for other in gathered[1:]:
                    expected = expected + other.float()
                expected = expected.to(torch.bfloat16)
                out = exchange(partial.clone())
                torch.cuda.synchronize()
                assert torch.equal(out.view(torch.int16), expected.view(torch.int16)), (call, rows)
                checked += 1
            ok, words = _lib.device_status()
            assert ok, words
            exchange.close()
            results[rank] = checked
        elif case == "graph":
            # The call number lives on the device, so a captured graph of several calls can be replayed.
            hidden, rows = 2048, 16
            exchange = tp.PeerAllReduce(device, rank, world, rows * hidden)
            partials = [synth.activations(500 + 10 * i + rank, rows, hidden, device) for i in range(4)]
            expected = []
            for partial in partials:
                gathered = [torch.empty_like(partial) for _ in range(world)]
                dist.all_gather(gathered, partial)
                total = gathered[0].float()
                for other in gathered[1:]:
                    total = total + other.float()
                expected.append(total.to(torch.bfloat16))
            buffers = [torch.empty_like(partial) for partial in partials]
            stream = torch.cuda.Stream(device)
            exchange(partials[0].clone())            # first call outside the graph (lazy set-up)
            torch.cuda.synchronize()
            dist.barrier()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(stream):
                with torch.cuda.graph(graph, stream=stream):
                    for buffer, partial in zip(buffers, partials):
                        buffer.copy_(partial)
                        exchange(buffer)
            torch.cuda.synchronize()
            for replay in range(5):
                with torch.cuda.stream(stream):
                    graph.replay()
                torch.cuda.synchronize()
                for index, (buffer, want) in enumerate(zip(buffers, expected)):
                    assert torch.equal(buffer.view(torch.int16), want.view(torch.int16)), (replay, index)
            ok, words = _lib.device_status()
            assert ok, words
            exchange.close()
            results[rank] = True
        elif case == "mlp":
            hidden, inter = 1024, 4096
            gate, up, down = synth.mlp_weights(77, hidden, inter)
            sharded = tp.TensorParallelMLP.from_full(gate, up, down, device, rank, world)
            move = lambda triple: tuple(t.to(device) for t in triple)  # noqa: E731
            gate, up, down = move(gate), move(up), move(down)
            worst = 0.0
            for rows in (1, 4, 16, 128):
                x = synth.activations(5 + rows, rows, hidden, device)
                r = synth.activations(6 + rows, rows, hidden, device)
                got = sharded(x, r)
                want = B.mlx_affine_mlp_executor(x, *gate, *up, *down, r)(x, r)
                torch.cuda.synchronize()
                peak = want.float().abs().max().item()
                error = (got.float() - want.float()).abs().max().item()
                assert error <= 6e-3 * peak, (rows, error / peak)
                worst = max(worst, error / peak)
                both = [torch.empty_like(got) for _ in range(world)]
                dist.all_gather(both, got)
                assert torch.equal(both[0].view(torch.int16), both[1].view(torch.int16)), rows
            tp.close_peer_groups()
            results[rank] = worst
        elif case == "late":
            exchange = tp.PeerAllReduce(device, rank, world, 4096, limit_ms=50)
            data = torch.full((4096,), float(rank + 1), dtype=torch.bfloat16, device=device)
            if rank == 0:
                out = exchange(data.clone())          # rank 1 has not called yet: the wait runs out
                ok, words = _lib.device_status()      # synchronises, reads and clears the record
                assert not ok and words[0] == 0x9E0 and words[2] == 1, words
                dist.barrier()                        # now let rank 1 make the same call
                dist.barrier()
                out = exchange(data.clone())          # the next call works again
                torch.cuda.synchronize()
                assert torch.all(out.float() == 3.0)
            else:
                dist.barrier()
                out = exchange(data.clone())          # finds rank 0's data already here
                torch.cuda.synchronize()
                assert torch.all(out.float() == 3.0)
                dist.barrier()
                out = exchange(data.clone())
                torch.cuda.synchronize()
                assert torch.all(out.float() == 3.0)
            ok, words = _lib.device_status()
            assert ok, words
            time.sleep(0.05)
            exchange.close()
            results[rank] = True
    finally:
        dist.destroy_process_group()


def _run(case):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    context = mp.get_context("spawn")
    results = context.Manager().dict()
    port = _free_port()
    children = [context.Process(target=_child, args=(rank, 2, port, case, results)) for rank in range(2)]
    for child in children:
        child.start()
    for child in children:
        child.join(180)
    for child in children:
        if child.is_alive():
            child.terminate()
            child.join(10)
            pytest.fail(f"{case}: a rank did not finish")
        assert child.exitcode == 0, f"{case}: rank exited with {child.exitcode}"
    return dict(results)


def test_peer_sum_equals_the_rank_order_sum_bit_for_bit():
    results = _run("sum")
    assert results == {0: 32, 1: 32}


def test_two_shot_exchange_gives_the_same_bits():
    """Reduce-scatter then all-gather through peer memory (the form very large messages among many
    ranks take), forced here on two ranks: same rank-order sums, bit for bit."""
    results = _run("sum_two_shot")
    assert results == {0: 32, 1: 32}


def test_sharded_mlp_matches_unsharded_and_is_identical_on_both_ranks():
    results = _run("mlp")
    assert set(results) == {0, 1}


def test_late_peer_makes_the_wait_run_out_and_the_next_call_recovers():
    results = _run("late")
    assert results == {0: True, 1: True}


def test_exchange_inside_a_replayed_cuda_graph():
    results = _run("graph")
    assert results == {0: True, 1: True}
