"""Per-direction edge weights from an image or an edge map, on the GPU.

Same names and arguments as the reference's utils/edge_weights.py (`get_steps` :5-42,
`getEdgeShift` :45-111, `multi_edge_weights` :114-179); the D shifted-difference passes of slicing
ops become one kernel (`mpl_edge_weights`) that writes all directions.  `edge_weights_native` is the
entry without the reference's shape conventions: its output for the channel-reducing modes is
already the layers' `edge_weights` [D,B,cv=1,H,W].
"""
import torch
import torch.nn.functional as F

from . import _lib

_STEPS = [(0, 1), (0, -1), (1, 0), (-1, 0), (1, 1), (-1, -1), (1, -1), (-1, 1), (1, 2), (-1, -2),
          (2, 1), (-2, -1), (2, -1), (-2, 1), (1, -2), (-1, 2)]

REDUCING_MODES = ("superpixel_edge", "kernel_cue_real", "kernel_cue_binary", "threshold", "cue_penalty")


def get_steps(dir):
    """(h_step, w_step) of direction `dir` (utils/edge_weights.py:5-42)."""
    if 0 <= dir < 16:
        return _STEPS[dir]
    print('Warning, edge weights support only 16 directions by far')
    return 0, 0


def edge_weights_native(edge_mode, image, n_dirs, sigma=10, threshold=0, penalty=0):
    """image: CUDA float32 [B,C,H,W].  Returns [n_dirs,B,Cout,H,W] with Cout = 1 for the modes in
    REDUCING_MODES, else C.  A mode name the reference does not know selects its fall-through
    branch (the image shifted by one step), as there."""
    _lib.require(image, "image", torch.float32)
    if image.dim() != 4:
        raise RuntimeError("image must be [B,C,H,W], got %s" % (tuple(image.shape),))
    if not 1 <= int(n_dirs) <= 16:
        raise RuntimeError("n_dirs must be in 1..16, got %d" % n_dirs)
    L = _lib.lib()
    mode = L.mpl_edge_mode(str(edge_mode).encode())
    if mode < 0:
        mode = L.mpl_edge_mode(b"shifted")
    b, c, h, w = image.shape
    cout = L.mpl_edge_mode_channels(mode, c)
    dev = image.device
    out = torch.empty(int(n_dirs), b, cout, h, w, dtype=torch.float32, device=dev)
    if out.numel() == 0:
        return out
    with torch.cuda.device(dev):
        ws = _lib.workspace(128, dev)
        _lib.check(L.mpl_edge_weights(mode, _lib.ptr(image), b, c, h, w, int(n_dirs), float(sigma),
                                      float(threshold), float(penalty), _lib.ptr(out), _lib.ptr(ws), 128,
                                      _lib.stream_ptr(dev)))
    return out


def getEdgeShift(edge_mode, image, n_dirs, sigma=10, threshold=0, penalty=0):
    """utils/edge_weights.py:45-111.  image (h,w), (channels,h,w) or (batch,channels,h,w); returns
    (n_dir,[batch,][channels,]h,w).  For the modes that reduce over channels the reference assigns
    a (batch,h,w) result into a (batch,channels,h,w) slot, which broadcasts only for batch == 1 (or
    channels == 1); the same restriction applies here and the value is repeated over channels."""
    n = image.dim()
    if n == 2:
        image = image.unsqueeze(0).unsqueeze(0)
    elif n == 3:
        image = image.unsqueeze(0)
    assert image.dim() == 4, image.size()
    image = image.contiguous().float()
    b, c, h, w = image.shape
    out = edge_weights_native(edge_mode, image, n_dirs, sigma=sigma, threshold=threshold, penalty=penalty)
    if out.size(2) != c:
        if b != 1 and c != 1:
            raise RuntimeError("edge_mode %s reduces over channels: the reference's assignment broadcasts "
                               "only for batch == 1 or channels == 1 (got batch %d, channels %d)" %
                               (edge_mode, b, c))
        out = out.repeat(1, 1, c, 1, 1)
    if n == 2:
        out = out.squeeze(1).squeeze(1)
    elif n == 3:
        out = out.squeeze(1)
    return out


def multi_edge_weights(edge_mode, img, n_dirs, scale_list=None, sigma=5, threshold=10, penalty=2,
                       padding_mask=None):
    """utils/edge_weights.py:114-179: one edge-weight tensor (n_dir,h*s,w*s) per scale s of
    `scale_list`, from img (channels,h,w).  Resampling is torch's, as in the reference."""
    groups, masks = [], []
    channel, height, width = img.size()
    use_mask = padding_mask is not None
    for scale in scale_list:
        h_size, w_size = int(height * scale), int(width * scale)
        if scale == 1:
            groups.append(img)
            if use_mask:
                masks.append(padding_mask)
            continue
        nearest = edge_mode in ['gt_edge', 'edge_net', 'edge_net_sigmoid', 'superpixel_edge']
        scaled = F.interpolate(img.unsqueeze(0), scale_factor=(scale, scale),
                               mode='nearest' if nearest else 'bilinear',
                               align_corners=None if nearest else True)
        groups.append(scaled.squeeze(0))
        if use_mask:
            w_grid = torch.linspace(-1, 1, w_size, device=img.device).repeat(h_size, 1)
            h_grid = torch.linspace(-1, 1, h_size, device=img.device).view(-1, 1).repeat(1, w_size)
            grid = torch.cat((w_grid.unsqueeze(2), h_grid.unsqueeze(2)), 2)
            m = F.grid_sample(padding_mask.unsqueeze(0), grid.unsqueeze(0))
            masks.append((m.squeeze(0) > 0.5).float())
    out = []
    for idx, scaled in enumerate(groups):
        if n_dirs > 0:
            shifted = getEdgeShift(edge_mode, scaled, n_dirs, sigma=sigma, threshold=threshold,
                                   penalty=penalty).squeeze(1)
        else:
            shifted = scaled
        if use_mask:
            shifted = shifted * masks[idx]
        if edge_mode == 'superpixel_edge':
            shifted = shifted[:, 0]
        out.append(shifted)
    return out
