"""TEST INFRASTRUCTURE ONLY -- Python reader of the Darknet-style cfg subset the library accepts; same keys and
defaults as the library's C reader, which follows dnn/NetworkFactory.c:77-173,328-354,543-601,671-824.
Describes a network to the CPU oracle (tests, the smoke check and the benchmark's CPU-baseline legs);
the product package never imports it."""

ACT = {"linear": 0, "relu": 1, "leaky": 2, "logistic": 3, "relu6": 4, "relie": 5, "ramp": 6, "tanh": 7, "plse": 8, "elu": 9,
       "loggy": 10, "hardtan": 11, "lhtan": 12, "selu": 13, "swish": 14, "mish": 15}
CONV, MAXPOOL, AVGPOOL, SOFTMAX, DROPOUT, SHORTCUT = 0, 1, 2, 3, 4, 5


def parse(text):
    secs = []
    for raw in text.splitlines():
        line = raw.strip()
        if not line or line[0] in "#;":
            continue
        if line.startswith("["):
            secs.append((line[1:line.index("]")].strip(), {}))
        else:
            k, v = line.split("=", 1)
            secs[-1][1][k.strip()] = v.strip()
    return secs


def network_spec(text, batch=0):
    """Returns (net options dict, list of layer dicts shaped like the oracle's aeto_layer_spec)."""
    secs = parse(text)
    name, ns = secs[0]
    assert name in ("net", "network")
    sub = int(ns.get("subdivisions", 1))
    net = dict(batch=int(ns.get("batch", 1)) // sub, subdivisions=sub, c=int(ns["channels"]), h=int(ns["height"]),
               w=int(ns["width"]), learning_rate=float(ns.get("learning_rate", .001)),
               momentum=float(ns.get("momentum", .9)), decay=float(ns.get("decay", .0001)))
    if batch:
        net["batch"], net["subdivisions"] = batch, 1
    layers = []
    for name, s in secs[1:]:
        if name in ("convolutional", "conv"):
            size = int(s.get("size", 1))
            stride = int(s.get("stride", 1))
            sx, sy = int(s.get("stride_x", -1)), int(s.get("stride_y", -1))
            sx = stride if sx < 1 else sx
            sy = stride if sy < 1 else sy
            padding = int(s.get("padding", 0))
            if int(s.get("pad", 0)):
                padding = size // 2
            layers.append(dict(type=CONV, filters=int(s.get("filters", 1)), size=size, stride_x=sx, stride_y=sy,
                               pad=padding, batch_normalize=int(s.get("batch_normalize", 0)),
                               activation=ACT[s.get("activation", "logistic")],
                               learning_rate_scale=float(s.get("learning_rate", 1))))
        elif name in ("maxpool", "max"):
            stride = int(s.get("stride", 1))
            size = int(s.get("size", stride))
            layers.append(dict(type=MAXPOOL, size=size, stride_x=int(s.get("stride_x", stride)),
                               stride_y=int(s.get("stride_y", stride)), pad=int(s.get("padding", size - 1))))
        elif name in ("avgpool", "avg"):
            layers.append(dict(type=AVGPOOL))
        elif name in ("softmax", "soft"):
            layers.append(dict(type=SOFTMAX, groups=int(s.get("groups", 1)), temperature=float(s.get("temperature", 1))))
        elif name == "dropout":
            layers.append(dict(type=DROPOUT, probability=float(s.get("probability", .2))))
        elif name == "shortcut":
            index = len(layers)
            src = [int(t) for t in s["from"].split(",") if t.strip()]
            layers.append(dict(type=SHORTCUT, activation=ACT[s.get("activation", "linear")],
                               **{"from": [i + index if i < 0 else i for i in src]}))
        else:
            raise ValueError("unsupported layer type [%s]" % name)
        # keys every layer type takes (dnn/NetworkFactory.c:926-934)
        layers[-1]["stopbackward"] = int(int(s.get("stopbackward", 0)) == 1)
        layers[-1]["dont_update"] = int(s.get("dont_update", 0))
    return net, layers
