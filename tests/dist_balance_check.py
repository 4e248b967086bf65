"""Two-rank check (gloo) of the vision-encoder data balance inside the Qwen2.5-VL model: rank 0 holds three images, rank 1
one; with ``model.encoder_balance`` the images are re-dealt before the vision tower and the embeddings come home, and
loss and every parameter gradient equal the run without it.  Run under torch.distributed.run; not collected by pytest."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from mindspeed_mm_b200.data.collate import PackedVLMCollator  # noqa: E402
from mindspeed_mm_b200.data.synthetic import SyntheticVLMDataset, SyntheticVLMSpec  # noqa: E402
from mindspeed_mm_b200.models.qwen2_5_vl import Qwen25VLConfig, Qwen25VLModel  # noqa: E402
from mindspeed_mm_b200.parallel.data_balance import EncoderBalance  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank = dist.get_rank()
    cfg = Qwen25VLConfig.tiny()
    cfg.text.num_layers, cfg.vision.depth, cfg.vision.fullatt_block_indexes = 1, 2, (1,)
    model = Qwen25VLModel(cfg).float()
    model.init_weights(0)
    n_img = 3 if rank == 0 else 1
    ds = SyntheticVLMDataset(SyntheticVLMSpec(seq_len=400, images_per_sample=n_img, image_size=112 if rank else 224,
                                              vocab_size=cfg.text.vocab_size, image_token_id=cfg.image_token_id,
                                              vision_start_token_id=cfg.vision_start_token_id, seed=7 + rank))
    batch = PackedVLMCollator.for_config(cfg)([ds[0]])

    def run(balance):
        model.zero_grad()
        model.encoder_balance = EncoderBalance(dist.group.WORLD) if balance else None
        loss_sum, n = model(batch)
        (loss_sum / n).backward()
        grads = {k: p.grad.clone() for k, p in model.named_parameters() if p.grad is not None}
        for g in grads.values():                      # vision gradients are spread over the ranks: compare the sums
            dist.all_reduce(g)
        return float((loss_sum / n).detach()), grads

    l0, g0 = run(False)
    l1, g1 = run(True)
    moved = model.encoder_balance.assign
    worst = max(float((g0[k] - g1[k]).abs().max()) for k in g0)
    ok = abs(l0 - l1) < 1e-5 and worst < 1e-5 and set(g0) == set(g1) and sorted(len(a) for a in moved) == [2, 2]
    flag = torch.tensor([int(ok)])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"dist_balance_check loss {l0:.6f} vs {l1:.6f} max grad diff {worst:.2e} assignment {moved} ok={bool(flag.item())}",
              flush=True)
    dist.destroy_process_group()
    sys.exit(0 if flag.item() else 1)


if __name__ == "__main__":
    main()
