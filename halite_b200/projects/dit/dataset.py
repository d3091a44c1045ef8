"""Image datasets for diffusion training (reference: projects/dit/dataset.py): a sorted
ImageFolder, record files holding encoded images with class ids, ADM-style centre cropping, and
a synthetic source for smoke tests."""

from __future__ import annotations

import io
import pickle

import numpy as np
import torch


def center_crop_arr(pil_image, image_size):
    """Halve with a box filter while at least twice too large, bicubic to the target short side,
    then crop the centre square (the ADM / guided-diffusion preprocessing)."""
    from PIL import Image

    while min(pil_image.size) >= 2 * image_size:
        pil_image = pil_image.resize(tuple(x // 2 for x in pil_image.size), resample=Image.Resampling.BOX)
    scale = image_size / min(pil_image.size)
    pil_image = pil_image.resize(tuple(round(x * scale) for x in pil_image.size), resample=Image.Resampling.BICUBIC)
    arr = np.array(pil_image)
    y, x = (arr.shape[0] - image_size) // 2, (arr.shape[1] - image_size) // 2
    return Image.fromarray(arr[y:y + image_size, x:x + image_size])


class CenterCrop:
    def __init__(self, image_size):
        self.image_size = image_size

    def __call__(self, img):
        return center_crop_arr(img, self.image_size)


class ToUint8Tensor:
    """PIL image -> uint8 [C, H, W] tensor (normalisation happens on the device)."""

    def __call__(self, img):
        return torch.from_numpy(np.array(img, dtype=np.uint8)).permute(2, 0, 1).contiguous()


def ImageFolder(*args, **kwargs):
    from torchvision import datasets

    ds = datasets.ImageFolder(*args, **kwargs)
    ds.samples = sorted(ds.samples)
    return ds


class RecordImageDataset:
    """Record file whose payloads are pickled `{"image": encoded bytes, "class_id": int}`."""

    def __init__(self, data_path: str, transform=None):
        from halite_b200.data.sources import FileInstruction, open_source

        self._reader = open_source([FileInstruction(data_path, 0, None, None)])
        self.transform = transform

    def __len__(self):
        return len(self._reader)

    def __getitem__(self, index):
        from PIL import Image

        rec = pickle.loads(self._reader[index])
        image = Image.open(io.BytesIO(rec["image"])).convert("RGB")
        if self.transform is not None:
            image = self.transform(image)
        return image, rec["class_id"]


BagzDataset = RecordImageDataset


class SyntheticImages(torch.utils.data.Dataset):
    """Class-dependent colour blobs: enough structure for a loss to fall, no files needed."""

    def __init__(self, n, image_size, n_labels=10, seed=0):
        self.n, self.image_size, self.n_labels, self.seed = n, image_size, n_labels, seed

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + i)
        label = i % self.n_labels
        base = torch.tensor([(label * 37) % 255, (label * 91) % 255, (label * 53) % 255], dtype=torch.float32)
        img = base.view(3, 1, 1) + 20 * torch.randn(3, self.image_size, self.image_size, generator=g)
        return img.clamp(0, 255).to(torch.uint8), label
