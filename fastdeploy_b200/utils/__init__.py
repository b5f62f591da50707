

def get_detection_test_image(path=None) -> str:
    """Path of a picture to try a detector on (python/fastdeploy/utils/example_resource.py:18-25). The reference downloads
    a photograph; without network access the file is taken from the local cache when it is there
    (``detection_test_image.jpg`` in ``FASTDEPLOY_MODEL_CACHE`` or in the resource directory), else a synthetic scene of
    coloured boxes on a gradient is drawn once and kept."""
    import os
    from . import hub_env
    from ..download import cache_dir
    name = "detection_test_image.jpg"
    path = path or hub_env.RESOURCE_HOME
    full = os.path.join(path, name)
    if os.path.exists(full):
        return full
    cached = os.path.join(cache_dir(), name)
    os.makedirs(path, exist_ok=True)
    if os.path.exists(cached):
        import shutil
        shutil.copyfile(cached, full)
        return full
    import cv2
    import numpy as np
    rng = np.random.default_rng(2023)
    h, w = 720, 1280
    yy, xx = np.mgrid[0:h, 0:w]
    img = np.stack([(xx * 255 // w), (yy * 255 // h), np.full((h, w), 96)], -1).astype(np.uint8)
    for _ in range(12):
        x0, y0 = int(rng.integers(0, w - 200)), int(rng.integers(0, h - 200))
        bw, bh = int(rng.integers(60, 200)), int(rng.integers(60, 200))
        cv2.rectangle(img, (x0, y0), (x0 + bw, y0 + bh), tuple(int(c) for c in rng.integers(0, 255, 3)), -1)
    cv2.imwrite(full, img)
    return full
