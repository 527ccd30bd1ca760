"""Data-parallel sharding of the MLP training step (one process per GPU, torch.distributed for the exchange).

The batch is split into contiguous row ranges, one per rank; each rank runs forward + backward over its range in chunks,
accumulating into its flat gradient arena with the MSE loss weighted so that the SUM over all chunks of all ranks is the
full-batch gradient; ONE all-reduce (sum) of the flat gradient arena follows, then the identical one-launch Adam step on
every replica. The reference has no multi-GPU path; per-replica semantics are those of its single-device training step
(zero_gradient, forward, mse::gradient, backward, step; tests/src/nn/cuda/cuda_basics.cu:922-929).
"""


def shard_range(n_rows: int, rank: int, world: int):
    """Contiguous, balanced row range [begin, end) of `rank` (the first n_rows % world ranks get one extra row)."""
    base, extra = divmod(n_rows, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def chunk_loss_weight(chunk_rows: int, total_rows: int) -> float:
    """mse::gradient divides by (rows * cols) of the chunk it is given (nn/loss_functions/mse/operations_generic.h:49);
    this weight turns that into a division by (total_rows * cols), so chunk gradients add up to the full-batch one."""
    return chunk_rows / float(total_rows)


def allreduce_sum_(tensor, dist=None, group=None):
    """In-place sum over ranks of a flat arena (NCCL over NVLink for CUDA tensors, gloo for CPU tensors)."""
    if dist is not None and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(tensor, op=dist.ReduceOp.SUM, group=group)
    return tensor


def sharded_train_step(pkg, net, x_shard, y_shard, total_rows: int, dist=None, group=None, exchange_events=None):
    """One optimizer step of `net` (rl_tools_b200.Mlp with batch == chunk size) on this rank's rows. x_shard / y_shard
    are CUDA tensors whose row count is a multiple of net.batch. exchange_events: an optional pair of CUDA events recorded
    on the current stream right before and right after the all-reduce, so that the exchange can be timed on its own."""
    rows = x_shard.shape[0]
    assert rows % net.batch == 0, "shard rows must be a multiple of the chunk size"
    net.zero_gradient()
    w = chunk_loss_weight(net.batch, total_rows)
    for c in range(0, rows, net.batch):
        x, y = x_shard[c:c + net.batch], y_shard[c:c + net.batch]
        out = net.forward(x)
        d_out = pkg.mse_gradient(out, y, w, d_a=net.d_out_buffer())
        net.backward(x, d_out)
    if exchange_events is not None:
        exchange_events[0].record()
    allreduce_sum_(net.grads, dist, group)
    if exchange_events is not None:
        exchange_events[1].record()
    net.step()
