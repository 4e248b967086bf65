"""Differentiable all-to-all along dim 0 with per-rank row counts (expert-parallel token exchange)."""
import torch
import torch.distributed as dist


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, group, input_, output_split_sizes, input_split_sizes):
        ctx.group, ctx.out_sizes, ctx.in_sizes = group, output_split_sizes, input_split_sizes
        world = dist.get_world_size(group=group)
        if world == 1:
            return input_
        input_ = input_.contiguous()
        if output_split_sizes is None:
            out = torch.empty_like(input_)
        else:
            out = input_.new_empty((int(sum(output_split_sizes)),) + tuple(input_.shape[1:]))
        dist.all_to_all_single(out, input_, output_split_sizes=output_split_sizes,
                               input_split_sizes=input_split_sizes, group=group)
        return out

    @staticmethod
    def backward(ctx, grad):
        return None, _AllToAll.apply(ctx.group, grad, ctx.in_sizes, ctx.out_sizes), None, None


def all_to_all(group, input_, output_split_sizes=None, input_split_sizes=None):
    if output_split_sizes is not None and not isinstance(output_split_sizes, list):
        output_split_sizes = [int(x) for x in output_split_sizes]
    if input_split_sizes is not None and not isinstance(input_split_sizes, list):
        input_split_sizes = [int(x) for x in input_split_sizes]
    return _AllToAll.apply(group, input_, output_split_sizes, input_split_sizes)
