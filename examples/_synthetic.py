"""Procedural data for the examples (there is no dataset download in them): seven-segment digit images, a two-moons
point cloud, and an embedded public-domain style text for the character models."""
import math

import torch

# segments: top, upper-left, upper-right, middle, lower-left, lower-right, bottom
_SEGMENTS = {0: "1110111", 1: "0010010", 2: "1011101", 3: "1011011", 4: "0111010", 5: "1101011", 6: "1101111",
             7: "1010010", 8: "1111111", 9: "1111011"}


def digit_images(n: int, size: int = 16, noise: float = 0.15, seed: int = 0):
    """n images [n, 1, size, size] of seven-segment digits, randomly shifted by up to two pixels with additive noise,
    and their labels [n]."""
    g = torch.Generator().manual_seed(seed)
    labels = torch.randint(0, 10, (n,), generator=g)
    imgs = torch.zeros(n, 1, size, size)
    a, b, m = 3, size - 4, size // 2                     # left / right (top / bottom) and the middle line
    for i, d in enumerate(labels.tolist()):
        on = _SEGMENTS[d]
        canvas = torch.zeros(size + 4, size + 4)
        def h(row): canvas[row + 2, a + 2:b + 3] = 1.0
        def v(col, r0, r1): canvas[r0 + 2:r1 + 3, col + 2] = 1.0
        if on[0] == "1": h(a)
        if on[1] == "1": v(a, a, m)
        if on[2] == "1": v(b, a, m)
        if on[3] == "1": h(m)
        if on[4] == "1": v(a, m, b)
        if on[5] == "1": v(b, m, b)
        if on[6] == "1": h(b)
        dy, dx = torch.randint(0, 5, (2,), generator=g).tolist()
        imgs[i, 0] = canvas[dy:dy + size, dx:dx + size]
    imgs += noise * torch.randn(imgs.shape, generator=g)
    return imgs, labels


def two_moons(n: int, noise: float = 0.05, seed: int = 0) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    t = torch.rand(n, generator=g) * math.pi
    upper = torch.rand(n, generator=g) < 0.5
    x = torch.where(upper, torch.cos(t), 1.0 - torch.cos(t))
    y = torch.where(upper, torch.sin(t), 0.5 - torch.sin(t))
    return torch.stack([x, y], 1) + noise * torch.randn(n, 2, generator=g)


TEXT = ("the quick brown fox jumps over the lazy dog. a journey of a thousand miles begins with a single step. "
        "all that glitters is not gold. the pen is mightier than the sword. practice makes perfect. "
        "actions speak louder than words. better late than never. every cloud has a silver lining. ") * 6
