"""Transform pipelines from a recipe's ``train_pipeline`` block: names and parameters of the reference's registry, shapes
and value ranges, and agreement with torchvision where both define the same operation."""
import torch

from mindspeed_mm_b200.data.transforms import (CenterCropResizeVideo, ResizeVideo, SpatialStrideCropVideo, TemporalRandomCrop,
                                               get_transforms, long_side_size, max_hw_size, resize_crop_to_fill)


def _clip(t=5, h=90, w=160):
    return (torch.rand(t, 3, h, w) * 255).to(torch.uint8)


def test_video_pipeline_from_recipe_block():
    # the pipeline of the reference's Wan2.1 T2V recipe
    block = {"video": [{"trans_type": "ToTensorVideo"},
                       {"trans_type": "CenterCropResizeVideo", "param": {"transform_size": "auto", "interpolation_mode": "bicubic",
                                                                         "antialias": True}},
                       {"trans_type": "ae_norm"}]}
    tf = get_transforms(True, block, transform_size={"max_height": 48, "max_width": 64})
    out = tf(_clip())
    assert out.shape == (5, 3, 48, 64) and out.dtype == torch.float32 and -1.3 <= float(out.min()) and float(out.max()) <= 1.3
    try:
        get_transforms(True, {"video": [{"trans_type": "NoSuchThing"}]})
        raise AssertionError
    except NotImplementedError:
        pass


def test_center_crop_resize_keeps_the_centre_and_the_ratio():
    clip = torch.zeros(1, 1, 100, 300)
    clip[..., :, 100:200] = 1.0                                    # the middle third is white
    out = CenterCropResizeVideo(transform_size={"max_height": 50, "max_width": 50})(clip)
    assert out.shape[-2:] == (50, 50) and float(out.mean()) > 0.99    # 1:1 crop of a 100 x 300 frame = the middle third
    top = CenterCropResizeVideo(transform_size=(50, 100), top_crop=True)(torch.arange(200.).view(1, 1, 200, 1).expand(1, 1, 200, 100))
    assert float(top[0, 0, 0, 0]) < 1.0                              # anchored at the top row


def test_resize_modes_and_helpers():
    assert long_side_size(720, 1280, (320, 640)) == (320, 568) and long_side_size(720, 1280, (480, 640)) == (360, 640)
    assert long_side_size(100, 100, (320, 640), skip_low_resolution=True) == (100, 100)
    assert max_hw_size(1000, 1000, 250000) == (500, 500) and max_hw_size(10, 10, 250000) == (10, 10)
    c = _clip(2, 72, 128).float()
    assert ResizeVideo({"max_height": 36, "max_width": 64}, mode="longside")(c).shape[-2:] == (36, 64)
    assert ResizeVideo({"max_hxw": 72 * 128 // 4}, mode="hxw")(c).shape[-2:] == (36, 64)
    assert SpatialStrideCropVideo(16)(_clip(1, 90, 170)).shape[-2:] == (80, 160)
    assert resize_crop_to_fill(c, (64, 64)).shape[-2:] == (64, 64)
    b, e = TemporalRandomCrop(16)(100)
    assert 0 <= b and e - b == 16 and e <= 100


def test_image_pipeline_matches_torchvision_resize():
    import torchvision.transforms as T
    from PIL import Image
    import numpy as np
    arr = (np.random.RandomState(0).rand(40, 60, 3) * 255).astype("uint8")
    img = Image.fromarray(arr)
    block = {"image": [{"trans_type": "ToTensor"}, {"trans_type": "Resize", "param": {"size": [20, 30], "interpolation": "BILINEAR"}},
                       {"trans_type": "norm_fun", "param": {"mean": [0.5, 0.5, 0.5], "std": [0.5, 0.5, 0.5]}}]}
    mine = get_transforms(False, block)(img)
    ref = T.Compose([T.ToTensor(), T.Resize([20, 30], interpolation=T.InterpolationMode.BILINEAR, antialias=True),
                     T.Normalize([0.5] * 3, [0.5] * 3)])(img)
    assert mine.shape == ref.shape == (3, 20, 30) and float((mine - ref).abs().max()) < 1e-5
    sq = get_transforms(False, {"image": [{"trans_type": "Pad2Square"}]})(img)
    assert sq.shape == (3, 60, 60) and torch.equal(sq[:, 10:50, :], torch.from_numpy(arr).permute(2, 0, 1))
