"""Model families under ZeRO-3 sharding (gloo): one optimizer step on W ranks equals the single-process step.

Covers the models whose forward reaches into several parameter containers (extra embedding tables, multiple heads,
two-stream blocks): every parameter access has to go through a sharding unit for this to hold."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mindspeed_mm_b200.api import stable_init_fn  # noqa: E402
from mindspeed_mm_b200.parallel.fsdp import FSDPEngine, OptimConfig  # noqa: E402
from mindspeed_mm_b200.parallel.state import init_parallel_state, reset_parallel_state  # noqa: E402


def _speech_samples():
    from mindspeed_mm_b200.data.synthetic import SyntheticSpeechDataset, SyntheticSpeechSpec
    ds = SyntheticSpeechDataset(SyntheticSpeechSpec(num_samples=4, text_len=6, frames=6))
    return [ds[0], ds[1]]


def cases():
    from mindspeed_mm_b200.models.diffusion import build_scheduler
    from mindspeed_mm_b200.models.ltx2 import LTX2Config, LTX2Model
    from mindspeed_mm_b200.models.omni import BagelConfig, BagelMoT, RewardModelBT
    from mindspeed_mm_b200.models.sdxl_unet import SDXLConfig, SDXLUNet
    from mindspeed_mm_b200.models.speech_lm import CosyVoice3LM, MultiCodebookLM, Qwen3TTSTalker
    from mindspeed_mm_b200.models.video_dits import JointDiT, VideoDiTConfig
    from mindspeed_mm_b200.models.wan import SoRAModel
    from mindspeed_mm_b200.models.wan_variants import VaceConfig, VaceWanDiT, Wan22Config, Wan22DiT
    from mindspeed_mm_b200.data.synthetic import SyntheticAVLatentDataset, SyntheticAVLatentSpec
    lat = dict(latents=torch.randn(1, 16, 2, 4, 4), prompt=torch.randn(1, 6, 64))
    av = SyntheticAVLatentDataset(SyntheticAVLatentSpec(num_samples=2))
    av_batch = {k: torch.stack([av[0][k], av[1][k]]) for k in av[0]}
    T = 14
    labels = torch.full((T,), -100)
    labels[[0, 1, 5, 6, 8]] = torch.tensor([3, 4, 5, 6, 7])
    bagel = dict(input_ids=torch.randint(1, 100, (T,)), text_rows=torch.tensor([0, 1, 2, 5, 6, 7, 8, 9]), vit_rows=torch.tensor([3, 4]),
                 vit_embeds=torch.randn(2, 24), latent_rows=torch.tensor([10, 11, 12, 13]), latents=torch.randn(4, 16),
                 latent_pos=torch.tensor([0, 1, 8, 9]), timesteps=torch.full((4,), 0.4), noise=torch.randn(4, 16),
                 position_ids=torch.cat([torch.arange(8), torch.arange(6)]), cu_seqlens=torch.tensor([0, 8, 14], dtype=torch.int32),
                 max_seqlen=8, labels=labels, loss_only=True)
    rm_batch = dict(input_ids=torch.randint(0, 1000, (10,)), position_ids=torch.cat([torch.arange(6), torch.arange(4)])[None].expand(3, -1),
                    cu_seqlens=torch.tensor([0, 6, 10], dtype=torch.int32), max_seqlen=6)

    def sora(net_fn, sched):
        def make():
            net = net_fn()
            with torch.device("cpu"):               # scheduler tables are data, not parameters: keep them off the meta device
                return SoRAModel(net, build_scheduler(sched), seed=0)
        return make

    return [
        ("moss_tts_delay", MultiCodebookLM, lambda m: m.collate(_speech_samples())),
        ("cosyvoice3", CosyVoice3LM, lambda m: m.eval().collate(_speech_samples())),
        ("qwen3tts", Qwen3TTSTalker, lambda m: m.collate(_speech_samples())),
        ("ltx2", lambda: LTX2Model(LTX2Config.tiny()), lambda m: av_batch),
        ("bagel", lambda: BagelMoT(BagelConfig.tiny()), lambda m: bagel),
        ("reward", RewardModelBT, lambda m: rm_batch),
        ("satdit", sora(lambda: JointDiT(VideoDiTConfig.tiny(in_channels=16, out_channels=16, text_dim=64)), dict(model_id="cogvideo_diffusion")),
         lambda m: lat),
        ("sdxl", sora(lambda: SDXLUNet(SDXLConfig.tiny()), dict(model_id="ddpm", learn_sigma=False, noise_schedule="scaled_linear")),
         lambda m: dict(latents=torch.randn(2, 4, 1, 8, 8), prompt=torch.randn(2, 6, 48),
                        added_cond=torch.cat([torch.randn(2, 24), torch.tensor([[64.0, 64.0, 0.0, 0.0, 64.0, 64.0]] * 2)], 1))),
        ("vace", sora(lambda: VaceWanDiT(VaceConfig.tiny()), dict(model_id="wan_flow_match_scheduler")),
         lambda m: dict(lat)),
        ("wan2_2_moe", sora(lambda: Wan22DiT(Wan22Config.tiny(moe_num_experts=2, per_token_timestep=True)), dict(model_id="wan_flow_match_scheduler")),
         lambda m: lat),
    ]


def run_case(factory, make_batch, group):
    torch.manual_seed(0)
    with torch.device("meta"):
        model = factory()
    eng = FSDPEngine(model.fsdp_units(), group=group, device="cpu", param_dtype=torch.float32,
                     opt=OptimConfig(lr=1e-2, weight_decay=0.0), no_recompute=())
    eng.materialize(stable_init_fn(0.05, 0))
    torch.manual_seed(1)
    batch = make_batch(model)
    if hasattr(model, "generator"):
        model.generator.manual_seed(0)
    eng.set_lr(1e-2)
    loss = model(batch, run=eng.run)
    loss.backward()
    eng.end_micro_step()
    eng.finish_step()
    return float(loss.detach()), {n: t.detach().clone() for n, t in eng.named_full_params()}


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    only = set(sys.argv[1:])
    ok_all = True
    torch.manual_seed(1234)                      # every rank draws the same batches
    for name, factory, make_batch in cases():
        if only and name not in only:
            continue
        ps = init_parallel_state(world_size=world, device_type="cpu")
        l_sh, got = run_case(factory, make_batch, ps.get_fsdp_group())
        reset_parallel_state()
        init_parallel_state(world_size=1, device_type="cpu")
        l_ref, ref = run_case(factory, make_batch, False)
        reset_parallel_state()
        worst = max((got[n] - t).abs().max().item() for n, t in ref.items()) if ref else 0.0
        ok = abs(l_sh - l_ref) < 1e-5 * max(1.0, abs(l_ref)) and worst < 5e-4 and set(got) == set(ref)
        ok_all &= ok
        if not ok and rank == 0:
            for n, t in ref.items():
                if n in got and (got[n] - t).abs().max().item() >= 5e-4:
                    print(f"    differs: {n} {tuple(t.shape)} by {(got[n] - t).abs().max().item():.2e}")
        if rank == 0:
            print(f"  {name}: loss {l_sh:.6f} vs {l_ref:.6f}, max param diff {worst:.2e}, {len(ref)} tensors -> {'ok' if ok else 'MISMATCH'}")
    f = torch.tensor([int(ok_all)])
    dist.all_reduce(f, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"dist_zoo_check world={world} ok={bool(f.item())}")
    dist.destroy_process_group()
    sys.exit(0 if f.item() else 1)


if __name__ == "__main__":
    main()
