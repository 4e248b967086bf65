"""Entry points beyond pre-training: inference, evaluation and post-training, driven by the same JSON / YAML trees.

The reference ships one script per task (inference_vlm.py:18, inference_sora.py:58, evaluate_vlm.py:20,
evaluate_gen.py:48, posttrain_sora_dpo.py:41, posttrain_flux_dancegrpo.py, pretrain_omni.py:24); the scripts at the
repository root call the functions below.  Every function takes an already parsed config dict, so it can be used
from Python as well; weights are random unless ``from_pretrained`` / ``load`` paths exist.
"""
from __future__ import annotations

import json
import os
from typing import Callable, Dict, List, Optional

import torch


def load_tree(path: str) -> dict:
    with open(path) as f:
        if path.endswith((".yaml", ".yml")):
            import yaml
            return yaml.safe_load(f)
        return json.load(f)


# ------------------------------------------------------------------------------------------ VLM inference / evaluation
def build_vlm_for_inference(cfg: dict, device="cpu", dtype=torch.float32):
    from ..checkpoint import hf as hfio
    from ..models.qwen2_5_vl import Qwen25VLConfig, Qwen25VLModel
    model_cfg = Qwen25VLConfig.from_mm_json(cfg["model"]) if "text_decoder" in cfg.get("model", {}) else \
        getattr(Qwen25VLConfig, cfg.get("model", {}).get("preset", "tiny"))()
    model = Qwen25VLModel(model_cfg)
    model.init_weights(int(cfg.get("seed", 0)))
    path = cfg.get("from_pretrained") or cfg.get("load")
    if path and os.path.exists(path) and hfio.is_hf_checkpoint(path):
        sd = hfio.to_internal(hfio.load_state_dict(path), hfio.qwen25vl_ops(model_cfg))
        own = model.state_dict()
        model.load_state_dict({k: v for k, v in sd.items() if k in own and own[k].shape == v.shape}, strict=False)
    return model.to(device=device, dtype=dtype).eval()


def _tokenizer(cfg):
    path = cfg.get("tokenizer") or cfg.get("from_pretrained")
    if path and os.path.exists(path):
        from transformers import AutoTokenizer
        return AutoTokenizer.from_pretrained(path)
    from ..data.multimodal import ByteTokenizer
    return ByteTokenizer()


def inference_vlm(cfg: dict, device="cpu") -> List[str]:
    """cfg: {"model": ..., "from_pretrained": dir, "prompts": [{"text": "...", "images": [paths]}], "max_new_tokens": n}."""
    from ..data.multimodal import ChatTemplate, Qwen2VLImageProcessor
    from ..tasks.inference import VLMGenerator
    model = build_vlm_for_inference(cfg, device)
    tok = _tokenizer(cfg)
    c = model.config
    sid = getattr(tok, "special_ids", None)
    if sid is not None and c.text.vocab_size >= tok.vocab_size:     # byte tokenizer: remap its specials onto the model's ids
        tmpl = ChatTemplate(tok, sid["<|image_pad|>"], sid["<|video_pad|>"], sid["<|vision_start|>"], sid["<|vision_end|>"])
        remap = {sid["<|image_pad|>"]: c.image_token_id, sid["<|vision_start|>"]: c.vision_start_token_id}
    else:
        tmpl = ChatTemplate(tok, c.image_token_id, getattr(c, "video_token_id", None), c.vision_start_token_id, None)
        remap = {}
    proc = Qwen2VLImageProcessor(patch_size=c.vision.patch_size, merge_size=c.vision.spatial_merge_size)
    gen = VLMGenerator(model, eos_token_id=cfg.get("eos_token_id"))
    outs = []
    for pr in cfg.get("prompts", []):
        rows, grids = [], []
        for path in pr.get("images", []):
            from PIL import Image
            r, g = proc(Image.open(path))
            rows.append(r)
            grids.append(g)
        counts = [g[0] * g[1] * g[2] // proc.merge ** 2 for g in grids]
        text = "<image>" * len(rows) + pr["text"] if "<image>" not in pr["text"] else pr["text"]
        ids, _ = tmpl.render([{"role": "user", "content": text}], counts, ["image"] * len(counts))
        ids += tmpl._enc("<|im_start|>assistant\n")
        ids = [remap.get(t, t) for t in ids]
        out = gen.generate(torch.tensor(ids), torch.cat(rows) if rows else None,
                           torch.tensor(grids) if grids else None, max_new_tokens=int(cfg.get("max_new_tokens", 16)), device=device)
        new = out[len(ids):].tolist()
        outs.append(tok.decode([t for t in new if t < getattr(tok, "vocab_size", 1 << 30)]) if hasattr(tok, "decode") else str(new))
    return outs


def evaluate_vlm(cfg: dict, device="cpu", predict: Optional[Callable[[dict], str]] = None) -> Dict[str, float]:
    """cfg: {"dataset": jsonl of {"question", "answer", "images"}, "metric": name, ...inference keys}."""
    from ..tasks.evaluation import evaluate
    with open(cfg["dataset"]) as f:
        samples = [json.loads(l) for l in f if l.strip()]
    if predict is None:
        def predict(s):
            one = dict(cfg, prompts=[{"text": s["question"], "images": s.get("images", [])}])
            return inference_vlm(one, device)[0]
    return evaluate(predict, samples, cfg.get("metric", "exact_match"))


# ------------------------------------------------------------------------------------------ video generation
def build_sora_for_inference(cfg: dict, device="cpu", dtype=torch.float32):
    from ..models.diffusion import build_scheduler
    from ..models.towers import build_ae, build_text_encoder
    from ..models.wan import WanConfig, WanDiT
    pred = dict(cfg["predictor"])
    if pred.get("model_id", "wandit") == "wandit":
        dit = WanDiT(WanConfig.from_mm_json(pred))
    else:
        from ..models.registry import build_model
        dit = build_model(pred["model_id"], pred)
    for p in dit.parameters():
        torch.nn.init.normal_(p, std=0.02)
    sched = build_scheduler(cfg.get("diffusion", {}))
    ae = build_ae(cfg.get("ae"), device, dtype)
    te = build_text_encoder(cfg.get("text_encoder"), device, dtype)
    return dit.to(device=device, dtype=dtype).eval(), sched, ae, te


def inference_sora(cfg: dict, device="cpu", out_dir: Optional[str] = None) -> List[torch.Tensor]:
    """cfg: model tree + {"prompts": [token-id lists or embeddings files], "frames", "height", "width", "save_path"}.
    Latent sizes are in latent units.  Returns the decoded videos (or latents when no VAE is configured)."""
    from ..tasks.inference import WanPipeline
    dit, sched, ae, te = build_sora_for_inference(cfg, device)
    pipe = WanPipeline(dit, sched, vae_decode=(lambda z: ae.decode(z)) if ae is not None else None)
    outs = []
    g = torch.Generator().manual_seed(int(cfg.get("seed", 0)))
    for i, pr in enumerate(cfg.get("prompts", [])):
        if isinstance(pr, str) and os.path.exists(pr):
            emb = torch.load(pr, map_location="cpu", weights_only=True)
        elif te is not None:
            emb = te.encode(torch.tensor([pr]).to(device))
        else:
            c = dit.config
            emb = torch.randn(1, c.text_len, c.text_dim, generator=g)
        v = pipe(emb, None, frames=int(cfg.get("frames", 3)), height=int(cfg.get("height", 8)), width=int(cfg.get("width", 8)),
                 generator=g, device=device)
        outs.append(v)
        save = out_dir or cfg.get("save_path")
        if save:
            os.makedirs(save, exist_ok=True)
            torch.save(v.cpu(), os.path.join(save, f"sample_{i:04d}.pt"))
            if v.shape[1] == 3:
                write_video(v[0], os.path.join(save, f"sample_{i:04d}.mp4"), fps=int(cfg.get("fps", 16)))
    return outs


def write_video(video: torch.Tensor, path: str, fps: int = 16) -> None:
    """video [3, T, H, W] in [-1, 1] -> mp4 through OpenCV."""
    import cv2
    x = ((video.float().clamp(-1, 1) + 1) * 127.5).byte().permute(1, 2, 3, 0).cpu().numpy()
    T, H, W, _ = x.shape
    wr = cv2.VideoWriter(path, cv2.VideoWriter_fourcc(*"mp4v"), fps, (W, H))
    for t in range(T):
        wr.write(cv2.cvtColor(x[t], cv2.COLOR_RGB2BGR))
    wr.release()


def evaluate_gen(cfg: dict, device="cpu", score_fn: Optional[Callable[[torch.Tensor, object], float]] = None) -> Dict[str, float]:
    """Generates one sample per prompt and aggregates ``score_fn(video, prompt)`` (the reference plugs VBench
    dimensions in here, evaluate_gen.py:48; without a scorer the temporal smoothness proxy below is reported)."""
    vids = inference_sora(cfg, device)

    def smooth(v, _):
        return float(1.0 - (v[:, :, 1:] - v[:, :, :-1]).abs().mean()) if v.shape[2] > 1 else 1.0
    fn = score_fn or smooth
    scores = [fn(v, p) for v, p in zip(vids, cfg.get("prompts", []))]
    return {"num_samples": len(scores), "score": sum(scores) / max(len(scores), 1)}


# ------------------------------------------------------------------------------------------ post-training
def posttrain_sora_dpo(cfg: dict, data_iter, device="cpu", steps: int = 1) -> List[Dict[str, float]]:
    import copy
    from ..tasks.posttrain import DiffusionDPOTrainer
    dit, sched, _, _ = build_sora_for_inference(cfg, device)
    dit.train()
    ref = copy.deepcopy(dit).eval().requires_grad_(False)
    opt = torch.optim.AdamW(dit.parameters(), lr=float(cfg.get("lr", 1e-6)), weight_decay=float(cfg.get("weight_decay", 0.0)))
    tr = DiffusionDPOTrainer(lambda x, t, c: dit(x, t, c), lambda x, t, c: ref(x, t, c), sched,
                             beta=float(cfg.get("dpo_beta", 5000.0)), optimizer=opt, seed=int(cfg.get("seed", 0)))
    return [tr.train_step(next(data_iter)) for _ in range(steps)]


def posttrain_flux_dancegrpo(cfg: dict, prompts, reward_fn, device="cpu", steps: int = 1) -> List[Dict[str, float]]:
    from ..models.diffusion import build_scheduler
    from ..models.mmdit import MMDiT, MMDiTConfig
    from ..tasks.posttrain import FlowGRPOTrainer
    pred = dict(cfg.get("predictor", {}))
    mc = MMDiTConfig.tiny() if pred.get("preset") == "tiny" else MMDiTConfig(**{k: tuple(v) if isinstance(v, list) else v
                                                                               for k, v in pred.items() if k not in ("model_id", "preset")})
    dit = MMDiT(mc).to(device)
    for p in dit.parameters():
        torch.nn.init.normal_(p, std=0.02)
    opt = torch.optim.AdamW(dit.parameters(), lr=float(cfg.get("lr", 1e-5)))
    sched = build_scheduler(cfg.get("diffusion", {}))
    g = cfg.get("grpo", {})
    tr = FlowGRPOTrainer(lambda x, t, c: dit(x, t, c[0].expand(x.shape[0], -1, -1), c[1].expand(x.shape[0], -1)), sched, reward_fn,
                         group_size=int(g.get("group_size", 4)), num_steps=int(g.get("num_steps", 8)), eta=float(g.get("eta", 0.3)),
                         clip_range=float(g.get("clip_range", 1e-4)), optimizer=opt, seed=int(cfg.get("seed", 0)))
    shape = (mc.in_channels, 1, int(g.get("height", 8)), int(g.get("width", 8)))
    return [tr.train_step(prompts[i % len(prompts)], shape, device) for i in range(steps)]
