"""Darknet cfg text for the detector architectures the benchmarks use, generated from compact
architecture descriptions (the reference keeps them as cfg/yolov3-tiny.cfg, cfg/yolov4.cfg and
cfg/yolov7.cfg; tests compare the generated networks with those files layer by layer when the
reference checkout is present).

Only inference-relevant keys are emitted: the cfg parser ignores training keys.
"""
from __future__ import annotations

ANCHORS_V4 = "12,16, 19,36, 40,28, 36,75, 76,55, 72,146, 142,110, 192,243, 459,401"
ANCHORS_V3_TINY = "10,14, 23,27, 37,58, 81,82, 135,169, 344,319"
_ACT = {"mi": "mish", "le": "leaky", "sw": "swish", "li": "linear", "lo": "logistic", "re": "relu"}


def _net(width, height, channels=3, batch=1):
    return "[net]\nbatch=%d\nsubdivisions=1\nwidth=%d\nheight=%d\nchannels=%d\n\n" % (batch, width, height, channels)


def _conv(filters, size, stride, act, bn=True):
    s = "[convolutional]\n"
    if bn:
        s += "batch_normalize=1\n"
    return s + "filters=%d\nsize=%d\nstride=%d\npad=1\nactivation=%s\n\n" % (filters, size, stride, act)


def _route(layers):
    return "[route]\nlayers=%s\n\n" % ",".join(str(v) for v in layers)


def _shortcut(frm, act="linear"):
    return "[shortcut]\nfrom=%d\nactivation=%s\n\n" % (frm, act)


def _maxpool(size, stride):
    return "[maxpool]\nsize=%d\nstride=%d\n\n" % (size, stride)


def _upsample(stride=2):
    return "[upsample]\nstride=%d\n\n" % stride


def _yolo(mask, anchors, classes, num, scale_x_y=None, new_coords=0):
    s = "[yolo]\nmask=%s\nanchors=%s\nclasses=%d\nnum=%d\n" % (",".join(str(m) for m in mask), anchors, classes, num)
    if scale_x_y is not None:
        s += "scale_x_y=%s\n" % scale_x_y
    if new_coords:
        s += "new_coords=1\n"
    return s + "\n"


def _expand(tokens: str, anchors: str, classes: int, num: int) -> str:
    """Token notation: c<filters>k<size>s<stride><act>[nb] | r[a,b,..] | s<from> | m<size>/<stride> | u<stride> |
    Y<mask>|<scale_x_y or ->|<new_coords>; act is a two-letter code (mi le sw li lo re), nb = no batch norm."""
    out = []
    for tok in tokens.split():
        if tok[0] == "c":
            f, rest = tok[1:].split("k")
            k, rest = rest.split("s", 1)
            stride, act = rest[0], rest[1:3]
            out.append(_conv(int(f), int(k), int(stride), _ACT[act], bn=not rest.endswith("nb")))
        elif tok[0] == "r":
            out.append(_route(int(v) for v in tok[2:-1].split(",")))
        elif tok[0] == "s":
            out.append(_shortcut(int(tok[1:])))
        elif tok[0] == "m":
            a, b = tok[1:].split("/")
            out.append(_maxpool(int(a), int(b)))
        elif tok[0] == "u":
            out.append(_upsample(int(tok[1:])))
        elif tok[0] == "Y":
            mask, sxy, nc = tok[1:].split("|")
            out.append(_yolo([int(m) for m in mask.split(",")], anchors, classes, num, None if sxy == "-" else sxy, int(nc)))
        else:
            raise ValueError(tok)
    return "".join(out)


def yolov3_tiny_cfg(width=416, height=416, batch=1, classes=80) -> str:
    head = "c%dk1s1linb" % (3 * (classes + 5))
    t = ("c16k3s1le m2/2 c32k3s1le m2/2 c64k3s1le m2/2 c128k3s1le m2/2 c256k3s1le m2/2 c512k3s1le m2/1 c1024k3s1le "
         "c256k1s1le c512k3s1le " + head + " Y3,4,5|-|0 r[-4] c128k1s1le u2 r[-1,8] c256k3s1le " + head + " Y0,1,2|-|0")
    return _net(width, height, 3, batch) + _expand(t, ANCHORS_V3_TINY, classes, 6)


def yolov4_cfg(width=608, height=608, batch=1, classes=80) -> str:
    """CSPDarknet53 (mish) + SPP + PANet (leaky), three heads with scale_x_y 1.2 / 1.1 / 1.05."""
    s = [_net(width, height, 3, batch)]
    s.append(_conv(32, 3, 1, "mish"))

    def csp_stage(out_ch, blocks, first):
        # down-sample, split into two 1x1 branches, residual blocks on one, concat, 1x1 merge
        s.append(_conv(out_ch, 3, 2, "mish"))
        part = out_ch if first else out_ch // 2
        hidden = out_ch // 2
        s.append(_conv(part, 1, 1, "mish"))
        s.append(_route([-2]))
        s.append(_conv(part, 1, 1, "mish"))
        for _ in range(blocks):
            s.append(_conv(hidden, 1, 1, "mish"))
            s.append(_conv(part, 3, 1, "mish"))
            s.append(_shortcut(-3))
        s.append(_conv(part, 1, 1, "mish"))
        s.append(_route([-1, -(3 * blocks + 4)]))
        s.append(_conv(out_ch, 1, 1, "mish"))

    csp_stage(64, 1, True)
    csp_stage(128, 2, False)
    csp_stage(256, 8, False)
    csp_stage(512, 8, False)
    csp_stage(1024, 4, False)
    head = "c%dk1s1linb" % (3 * (classes + 5))
    neck = ("c512k1s1le c1024k3s1le c512k1s1le m5/1 r[-2] m9/1 r[-4] m13/1 r[-1,-3,-5,-6] c512k1s1le c1024k3s1le c512k1s1le "
            "c256k1s1le u2 r[85] c256k1s1le r[-1,-3] c256k1s1le c512k3s1le c256k1s1le c512k3s1le c256k1s1le "
            "c128k1s1le u2 r[54] c128k1s1le r[-1,-3] c128k1s1le c256k3s1le c128k1s1le c256k3s1le c128k1s1le "
            "c256k3s1le " + head + " Y0,1,2|1.2|0 "
            "r[-4] c256k3s2le r[-1,-16] c256k1s1le c512k3s1le c256k1s1le c512k3s1le c256k1s1le c512k3s1le " + head + " Y3,4,5|1.1|0 "
            "r[-4] c512k3s2le r[-1,-37] c512k1s1le c1024k3s1le c512k1s1le c1024k3s1le c512k1s1le c1024k3s1le " + head + " Y6,7,8|1.05|0")
    s.append(_expand(neck, ANCHORS_V4, classes, 9))
    return "".join(s)


def yolov7_cfg(width=640, height=640, batch=1, classes=80) -> str:
    """E-ELAN backbone + SPPCSPC + ELAN-PAN neck (swish), three logistic heads decoded with new_coords=1, scale_x_y=2."""
    head = "c%dk1s1lonb" % (3 * (classes + 5))

    def elan(c, deep):  # two 1x1 branches, four 3x3 convs, concat of four taps, 1x1 merge
        return "c%dk1s1sw r[-2] c%dk1s1sw c%dk3s1sw c%dk3s1sw c%dk3s1sw c%dk3s1sw r[-1,-3,-5,-7] c%dk1s1sw " % (c, c, c, c, c, c, deep)

    def down(c):  # max-pool branch + strided-conv branch, concat
        return "m2/2 c%dk1s1sw r[-3] c%dk1s1sw c%dk3s2sw r[-1,-4] " % (c, c, c)

    def elan_w(c, half, out):  # neck ELAN: six taps
        return ("c%dk1s1sw r[-2] c%dk1s1sw c%dk3s1sw c%dk3s1sw c%dk3s1sw c%dk3s1sw r[-1,-2,-3,-4,-5,-7] c%dk1s1sw "
                % (c, c, half, half, half, half, out))

    t = "c32k3s1sw c64k3s2sw c64k3s1sw c128k3s2sw " + elan(64, 256)
    t += down(128) + elan(128, 512)
    t += down(256) + elan(256, 1024)
    t += down(512) + elan(256, 1024)
    # SPPCSPC
    t += ("c512k1s1sw r[-2] c512k1s1sw c512k3s1sw c512k1s1sw m5/1 r[-2] m9/1 r[-4] m13/1 r[-6,-5,-3,-1] c512k1s1sw c512k3s1sw "
          "r[-1,-13] c512k1s1sw ")
    t += "c256k1s1sw u2 r[42] c256k1s1sw r[-1,-3] " + elan_w(256, 128, 256)
    t += "c128k1s1sw u2 r[27] c128k1s1sw r[-1,-3] " + elan_w(128, 64, 128)
    t += "m2/2 c128k1s1sw r[-3] c128k1s1sw c128k3s2sw r[-1,-4,86] " + elan_w(256, 128, 256)
    t += "m2/2 c256k1s1sw r[-3] c256k1s1sw c256k3s2sw r[-1,-4,72] " + elan_w(512, 256, 512)
    t += "r[100] c256k3s1sw " + head + " Y0,1,2|2.0|1 r[115] c512k3s1sw " + head + " Y3,4,5|2.0|1 r[130] c1024k3s1sw " + head + " Y6,7,8|2.0|1"
    return _net(width, height, 3, batch) + _expand(t, ANCHORS_V4, classes, 9)


def head_specs(cfg_text: str):
    """[yolo] / [gaussian_yolo] parameters of a cfg as the decode API takes them: list of dicts {classes, anchors [(w,h)..], scale_x_y,
    new_coords} in layer order."""
    specs = []
    cur = None
    for raw in cfg_text.splitlines():
        line = raw.split("#")[0].strip()
        if not line:
            continue
        if line.startswith("["):
            cur = {} if line.strip("[]").strip().lower() in ("yolo", "gaussian_yolo") else None
            if cur is not None:
                specs.append(cur)
            continue
        if cur is not None and "=" in line:
            k, v = (p.strip() for p in line.split("=", 1))
            cur[k.lower()] = v
    out = []
    for d in specs:
        anchors = [float(v) for v in d["anchors"].replace(",", " ").split()]
        mask = [int(v) for v in d["mask"].replace(",", " ").split()]
        out.append(dict(classes=int(d.get("classes", 20)), anchors=[(anchors[2 * m], anchors[2 * m + 1]) for m in mask],
                        scale_x_y=float(d.get("scale_x_y", 1.0)), new_coords=int(d.get("new_coords", 0))))
    return out
