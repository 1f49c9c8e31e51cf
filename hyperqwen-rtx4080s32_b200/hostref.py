"""Host-side (numpy) statement of the packed layout, driven by the C ABI's slab map.  Used to check the
repack kernels and to inspect packed buffers; not a compute path."""
from __future__ import annotations

import numpy as np

from . import formats as F


def repack_numpy(raw: np.ndarray, wtype: int, slab_map: np.ndarray) -> np.ndarray:
    """raw uint8 [n_out, nb * B] -> tiles uint8 [ceil(n_out/64), nb, 64 * B] (rows past n_out zero)."""
    bb = F.BYTES_PER_256[wtype]
    n_out, nb = raw.shape[0], raw.shape[1] // bb
    n_tiles = -(-n_out // 64)
    padded = np.zeros((n_tiles * 64, nb, bb), np.uint8)
    padded[:n_out] = raw.reshape(n_out, nb, bb)
    # [tile, slab, row16, kb, byte] -> [tile, kb, slab, row16 * B + byte] -> permute by the map
    img = padded.reshape(n_tiles, 4, 16, nb, bb).transpose(0, 3, 1, 2, 4).reshape(n_tiles, nb, 4, 16 * bb)
    return np.ascontiguousarray(img[..., slab_map]).reshape(n_tiles, nb, 64 * bb)


def unrepack_numpy(tiles: np.ndarray, n_out: int, wtype: int, slab_map: np.ndarray) -> np.ndarray:
    bb = F.BYTES_PER_256[wtype]
    n_tiles, nb = tiles.shape[0], tiles.shape[1]
    img = np.empty((n_tiles, nb, 4, 16 * bb), np.uint8)
    img[..., slab_map] = tiles.reshape(n_tiles, nb, 4, 16 * bb)
    rows = img.reshape(n_tiles, nb, 4, 16, bb).transpose(0, 2, 3, 1, 4).reshape(n_tiles * 64, nb * bb)
    return np.ascontiguousarray(rows[:n_out])
