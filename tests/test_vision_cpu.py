"""Vision registry: every model family of the reference constructs and runs a forward on CPU."""
import pytest
import torch

from ferrotorch_b200 import vision

tv = pytest.mark.skipif(not vision.HAVE_TORCHVISION, reason="torchvision not installed")


def test_registry_lists_every_family():
    names = vision.available()
    for n in ["resnet18", "resnet50", "vgg16", "vit_b_16", "efficientnet_b0", "convnext_tiny", "swin_t", "mobilenet_v2",
              "densenet121", "inception_v3", "faster_rcnn", "mask_rcnn", "retinanet", "fcos", "ssd300", "deeplabv3",
              "fcn", "lraspp", "unet"]:
        assert n in names, n


@tv
@pytest.mark.parametrize("name,size", [("vgg11", 64), ("mobilenet_v2", 64), ("densenet121", 64), ("convnext_tiny", 64),
                                       ("efficientnet_b0", 64), ("swin_t", 64), ("vit_b_16", 224)])
def test_classifiers_forward(name, size):
    m = vision.build(name, num_classes=7).eval()
    with torch.no_grad():
        assert m(torch.randn(1, 3, size, size)).shape == (1, 7)


@tv
def test_segmenters_and_unet_forward():
    x = torch.randn(1, 3, 64, 64)
    with torch.no_grad():
        assert vision.build("fcn", num_classes=5).eval()(x)["out"].shape == (1, 5, 64, 64)
        assert vision.build("lraspp", num_classes=5).eval()(x)["out"].shape == (1, 5, 64, 64)
        assert vision.build("unet", num_classes=3, base=8, depth=3).eval()(x).shape == (1, 3, 64, 64)
        assert vision.build("unet", num_classes=3, base=8, depth=3).eval()(torch.randn(1, 3, 50, 70)).shape == (1, 3, 50, 70)


@tv
def test_detector_and_ops():
    m = vision.build("retinanet", num_classes=4).eval()
    with torch.no_grad():
        out = m([torch.rand(3, 128, 128)])
    assert set(out[0]) == {"boxes", "scores", "labels"}
    boxes = torch.tensor([[0.0, 0, 10, 10], [1, 1, 11, 11], [50, 50, 60, 60]])
    keep = vision.nms(boxes, torch.tensor([0.9, 0.8, 0.7]), 0.5)
    assert keep.tolist() == [0, 2]
    assert vision.box_iou(boxes[:1], boxes[:1]).item() == pytest.approx(1.0)
    feats = torch.arange(16.0).view(1, 1, 4, 4)
    assert vision.roi_align(feats, [torch.tensor([[0.0, 0, 4, 4]])], output_size=2).shape == (1, 1, 2, 2)


def test_own_resnet_keys_match_torchvision():
    if not vision.HAVE_TORCHVISION:
        pytest.skip("torchvision not installed")
    import torchvision

    ours = vision.build("resnet50").state_dict()
    theirs = torchvision.models.resnet50(weights=None).state_dict()
    assert set(ours) == set(theirs)
    assert all(ours[k].shape == theirs[k].shape for k in ours)


@pytest.mark.parametrize("name", ["resnet18", "resnet50"])
def test_own_resnet_computes_what_torchvision_computes(name):
    """Same weights, same input -> same logits (train and eval mode), same running statistics and
    the same gradients: the fused BN + residual + ReLU blocks are a re-arrangement, not a new model."""
    if not vision.HAVE_TORCHVISION:
        pytest.skip("torchvision not installed")
    import torchvision

    torch.manual_seed(0)
    theirs = getattr(torchvision.models, name)(weights=None)
    ours = vision.build(name)
    ours.load_state_dict(theirs.state_dict())
    x = torch.randn(4, 3, 64, 64)
    y = torch.randint(0, 1000, (4,))
    for mode in ("train", "eval"):
        getattr(theirs, mode)()
        getattr(ours, mode)()
        a, b = theirs(x), ours(x).float()
        assert torch.allclose(a, b, atol=2e-4, rtol=1e-4), (mode, (a - b).abs().max())
    k = "layer2.0.bn1.running_var"
    assert torch.allclose(theirs.state_dict()[k], ours.state_dict()[k], atol=1e-5)
    theirs.train(), ours.train()
    torch.nn.functional.cross_entropy(theirs(x), y).backward()
    torch.nn.functional.cross_entropy(ours(x).float(), y).backward()
    ga, gb = dict(theirs.named_parameters()), dict(ours.named_parameters())
    for k in ("conv1.weight", "layer1.0.bn1.weight", "layer3.1.conv2.weight", "fc.bias"):
        assert torch.allclose(ga[k].grad, gb[k].grad, atol=5e-4, rtol=1e-3), (k, (ga[k].grad - gb[k].grad).abs().max())


def test_image_io_and_extra_transforms(tmp_path):
    pytest.importorskip("PIL")
    torch.manual_seed(0)
    img = torch.rand(3, 9, 7)
    p = tmp_path / "a.png"
    vision.write_tensor_as_image(str(p), img)
    raw = vision.read_image(str(p))
    assert (raw.width, raw.height, raw.channels, len(raw.data)) == (7, 9, 3, 7 * 9 * 3)
    back = vision.read_image_as_tensor(str(p))
    assert back.shape == (3, 9, 7) and (back - img).abs().max() <= 0.5 / 255 + 1e-6        # PNG is lossless: only the rounding
    rgba = vision.read_image_rgba(str(p))
    assert rgba.channels == 4 and vision.raw_image_to_tensor(rgba)[3].min() == 1.0           # opaque alpha
    vision.write_image(str(tmp_path / "b.jpg"), rgba)                                        # alpha dropped for JPEG
    assert vision.read_image(str(tmp_path / "b.jpg")).channels == 3
    assert vision.tensor_to_raw_image(torch.tensor([[[2.0]], [[-1.0]], [[0.5]]])).data == bytes([255, 0, 128])
    for bad in (torch.zeros(9, 7), torch.zeros(2, 9, 7)):
        with pytest.raises(ValueError):
            vision.tensor_to_raw_image(bad)
    with pytest.raises(ValueError):
        vision.RawImage(b"123", 2, 2, 3)
    with pytest.raises(OSError):
        vision.read_image(str(tmp_path / "missing.png"))
    assert torch.equal(vision.VisionToTensor()(raw), back)
    n = vision.VisionNormalize([0.5, 0.5, 0.5], [0.25, 0.5, 1.0])(torch.full((3, 2, 2), 1.0))
    assert n[:, 0, 0].tolist() == [2.0, 1.0, 0.5]
    with pytest.raises(ValueError):
        vision.VisionNormalize([0.0], [0.0])
    vision.vision_manual_seed(7)
    a = vision.GaussianNoise(sigma=0.2)(img)
    vision.vision_manual_seed(7)
    b = vision.GaussianNoise(sigma=0.2)(img)
    assert torch.equal(a, b) and not torch.equal(a, img) and 0 <= a.min() and a.max() <= 1
    blur = vision.RandomGaussianBlur(5, (1.0, 1.0), p=1.0)(img)
    assert blur.shape == img.shape and blur.var() < img.var() and abs(float(blur.mean() - img.mean())) < 0.02
    assert torch.equal(vision.RandomGaussianBlur(3, p=0.0)(img), img)
    with pytest.raises(ValueError):
        vision.RandomGaussianBlur(4)


def test_reference_vision_names():
    import ferrotorch_b200.vision as V

    assert V.SSD_TOTAL_ANCHORS == 8732 and V.IMAGENET_MEAN == (0.485, 0.456, 0.406) and V.Split.Train.train
    assert V.get_model("resnet18", num_classes=5)(torch.randn(1, 3, 64, 64)).shape == (1, 5)
    reg = V.ModelRegistry()
    reg.register("tiny", lambda **kw: torch.nn.Linear(2, 2))
    assert reg.contains("tiny") and reg.contains("faster_rcnn") and isinstance(reg.get("tiny"), torch.nn.Linear)
    with pytest.raises(ValueError):
        reg.register("resnet50", lambda: None)
    net = V.ResNet50Dilated(num_classes=3)
    feats = V.create_feature_extractor(net, {"layer2": "c3", "layer4": "c5"})(torch.randn(1, 3, 64, 64))
    assert feats["c3"].shape[-1] == 8 and feats["c5"].shape[-1] == 8 and feats["c5"].shape[1] == 2048   # stride stays 8
    seg = V.fcn_resnet50(num_classes=4).eval()
    assert isinstance(seg, V.Fcn) and seg(torch.randn(1, 3, 64, 64))["out"].shape == (1, 4, 64, 64)
    assert V.Resize(8)(torch.rand(3, 16, 16)).shape == (3, 8, 8) and V.CenterCrop(4)(torch.rand(3, 8, 8)).shape == (3, 4, 4)
    rpn = V.RpnConfig(nms_thresh=0.6).build(V.AnchorGenerator(((32,),), ((1.0,),)), V.RpnHead(8, 1))
    assert isinstance(rpn, V.Rpn) and rpn.nms_thresh == 0.6


# --------------------------------------------------------------------------- own model zoo vs torchvision
def _same_as_torchvision(ours, tv, x, get=lambda o: o):
    tv.eval(), ours.eval()
    ours.load_state_dict(tv.state_dict(), strict=True)          # torchvision's parameter names
    with torch.no_grad():
        torch.testing.assert_close(get(ours(x)), get(tv(x)), rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("name", ["vgg11", "mobilenet_v2", "convnext_tiny", "densenet121"])
def test_own_classifiers_match_torchvision(name):
    tvm = pytest.importorskip("torchvision.models")
    from ferrotorch_b200.models import vision_zoo as Z

    torch.manual_seed(0)
    _same_as_torchvision(getattr(Z, name)(num_classes=7), getattr(tvm, name)(weights=None, num_classes=7),
                         torch.randn(2, 3, 64, 64))


def test_own_vit_matches_torchvision_and_trains():
    tvm = pytest.importorskip("torchvision.models")
    from ferrotorch_b200.models import vision_zoo as Z

    torch.manual_seed(1)
    ours = Z.VisionTransformer(image_size=32, patch_size=8, num_layers=2, num_heads=4, hidden_dim=64, mlp_dim=128, num_classes=5)
    tv = tvm.VisionTransformer(image_size=32, patch_size=8, num_layers=2, num_heads=4, hidden_dim=64, mlp_dim=128, num_classes=5)
    _same_as_torchvision(ours, tv, torch.randn(3, 3, 32, 32))
    ours.train()
    ours(torch.randn(2, 3, 32, 32)).sum().backward()
    assert all(p.grad is not None for p in ours.parameters())


@pytest.mark.parametrize("name", ["fcn_resnet50", "deeplabv3_resnet50"])
def test_own_segmentation_models_match_torchvision(name):
    seg = pytest.importorskip("torchvision.models.segmentation")
    from ferrotorch_b200.models import vision_zoo as Z

    torch.manual_seed(2)
    _same_as_torchvision(getattr(Z, name)(num_classes=4),
                         getattr(seg, name)(weights=None, weights_backbone=None, num_classes=4, aux_loss=False),
                         torch.randn(2, 3, 64, 64), lambda o: o["out"])


@pytest.mark.parametrize("name,size", [("efficientnet_b0", (64, 64)), ("mobilenet_v3_large", (64, 64)),
                                       ("mobilenet_v3_small", (64, 64)), ("inception_v3", (139, 139)), ("swin_t", (100, 84))])
def test_own_classifier_families_match_torchvision(name, size):
    # sizes that are not multiples of the window / stride exercise Swin's padding, shift masks and patch merging
    tvm = pytest.importorskip("torchvision.models")
    from ferrotorch_b200.models import vision_families as Z

    torch.manual_seed(3)
    kw = {"init_weights": False} if name == "inception_v3" else {}
    _same_as_torchvision(getattr(Z, name)(num_classes=7), getattr(tvm, name)(weights=None, num_classes=7, **kw),
                         torch.randn(2, 3, *size))


def test_own_lraspp_matches_torchvision_and_families_train():
    seg = pytest.importorskip("torchvision.models.segmentation")
    from ferrotorch_b200.models import vision_families as Z

    torch.manual_seed(4)
    _same_as_torchvision(Z.lraspp_mobilenet_v3_large(num_classes=5),
                         seg.lraspp_mobilenet_v3_large(weights=None, weights_backbone=None, num_classes=5),
                         torch.randn(2, 3, 96, 80), lambda o: o["out"])
    # training mode: stochastic depth, dropout and the auxiliary classifier are live, every parameter gets a gradient
    net = Z.inception_v3(num_classes=3).train()
    out, aux = net(torch.randn(2, 3, 299, 299))
    (out.sum() + aux.sum()).backward()
    assert all(p.grad is not None for p in net.parameters())
    swin = Z.SwinTransformer(embed_dim=24, depths=(2, 2), heads=(2, 4), window=4, num_classes=3).train()
    swin(torch.randn(2, 3, 40, 40)).sum().backward()
    assert all(p.grad is not None for p in swin.parameters())


def test_own_detection_operators_match_torchvision():
    O = pytest.importorskip("torchvision.ops")
    from ferrotorch_b200.ops import det_ops as D

    torch.manual_seed(5)

    def rb(n, s=100.0):
        xy, wh = torch.rand(n, 2) * s, torch.rand(n, 2) * s / 2 + 1
        return torch.cat([xy, xy + wh], 1)

    a, b, sc, idx = rb(50), rb(40), torch.rand(50), torch.randint(0, 3, (50,))
    assert torch.allclose(D.box_iou(a, b), O.box_iou(a, b), atol=1e-6)
    for t in (0.3, 0.5, 0.7):
        assert torch.equal(D.nms(a, sc, t), O.nms(a, sc, t))              # sweep in the native host library
        assert torch.equal(D.nms_torch(a, sc, t), O.nms(a, sc, t))        # torch formulation
    assert D._host_lib() is not None, "the native host library must be the path that runs"
    assert torch.equal(D.batched_nms(a, sc, idx, 0.5), O.batched_nms(a, sc, idx, 0.5))
    feat = torch.randn(2, 5, 20, 24)
    rois = torch.cat([torch.randint(0, 2, (30, 1)).float(), rb(30, 80)], 1)
    rois[0, 1:] = torch.tensor([-20.0, -10.0, 5.0, 8.0])       # partly outside
    rois[1, 1:] = torch.tensor([70.0, 60.0, 120.0, 130.0])     # beyond the far edge
    rois[2, 1:] = torch.tensor([10.0, 10.0, 10.2, 10.1])       # smaller than one pixel
    for aligned in (False, True):
        for scale in (0.25, 1.0):
            torch.testing.assert_close(D.roi_align(feat, rois, 7, scale, 2, aligned), O.roi_align(feat, rois, 7, scale, 2, aligned),
                                       atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(D.roi_align(feat, rois, (3, 5), 0.5, 3), O.roi_align(feat, rois, (3, 5), 0.5, 3), atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(D.roi_align_torch(feat, rois, 7, 0.25, 2, True), O.roi_align(feat, rois, 7, 0.25, 2, True), atol=1e-5, rtol=1e-5)
    fr = feat.clone().requires_grad_()                                  # under autograd: the torch formulation, with a gradient
    ft_ = feat.clone().requires_grad_()
    D.roi_align(fr, rois, 7, 0.5, 2).square().sum().backward()
    O.roi_align(ft_, rois, 7, 0.5, 2).square().sum().backward()
    torch.testing.assert_close(fr.grad, ft_.grad, atol=1e-4, rtol=1e-4)
    feats = {str(i): torch.randn(2, 4, 64 >> i, 64 >> i) for i in range(4)}
    boxes = [rb(20, 200), rb(15, 200)]
    boxes[0][0], boxes[1][0] = torch.tensor([0.0, 0.0, 255.0, 255.0]), torch.tensor([5.0, 5.0, 9.0, 9.0])
    want = O.MultiScaleRoIAlign(["0", "1", "2", "3"], 7, 2)(feats, boxes, [(256, 256), (256, 256)])
    torch.testing.assert_close(D.MultiScaleRoIAlign(["0", "1", "2", "3"], 7, 2)(feats, boxes, (256, 256)), want, atol=1e-5, rtol=1e-5)


def _same_detections(ours, tv, x, keys=("boxes", "scores", "labels")):
    tv.eval(), ours.eval()
    sd = tv.state_dict()
    for k, v in sd.items():                                   # non-trivial batch-norm statistics
        if k.endswith("running_mean"):
            v.normal_(0, 0.1)
        elif k.endswith("running_var"):
            v.uniform_(0.5, 1.5)
    ours.load_state_dict(sd, strict=True)                      # torchvision's parameter names
    with torch.no_grad():
        got, want = ours(x), tv(list(x))
    for g, w in zip(got, want):
        assert len(g["boxes"]) > 0
        for k in keys:
            if g[k].dtype.is_floating_point:
                torch.testing.assert_close(g[k], w[k], atol=2e-3, rtol=1e-3)
            else:
                assert torch.equal(g[k], w[k])


@pytest.mark.parametrize("name", ["fasterrcnn", "maskrcnn", "keypointrcnn", "retinanet", "fcos", "ssd300"])
def test_own_detectors_match_torchvision(name):
    # same weights, identity input transform on torchvision's side: proposals, scores, labels, masks and keypoints agree
    TD = pytest.importorskip("torchvision.models.detection")
    from ferrotorch_b200.models import detection as M

    torch.manual_seed(6)
    ident = dict(weights=None, weights_backbone=None, image_mean=[0.0, 0.0, 0.0], image_std=[1.0, 1.0, 1.0])
    sized = dict(min_size=128, max_size=160, **ident)
    x = torch.rand(2, 3, 128, 160)
    if name == "fasterrcnn":
        _same_detections(M.fasterrcnn_resnet50_fpn(5), TD.fasterrcnn_resnet50_fpn(num_classes=5, **sized), x)
    elif name == "maskrcnn":
        _same_detections(M.maskrcnn_resnet50_fpn(5), TD.maskrcnn_resnet50_fpn(num_classes=5, **sized), x,
                         ("boxes", "scores", "labels", "masks"))
    elif name == "keypointrcnn":
        _same_detections(M.keypointrcnn_resnet50_fpn(2, 17), TD.keypointrcnn_resnet50_fpn(num_classes=2, num_keypoints=17, **sized),
                         x, ("boxes", "scores", "labels", "keypoints", "keypoints_scores"))
    elif name == "retinanet":
        _same_detections(M.retinanet_resnet50_fpn(5, score_thresh=0.0),
                         TD.retinanet_resnet50_fpn(num_classes=5, score_thresh=0.0, **sized), x)
    elif name == "fcos":
        _same_detections(M.fcos_resnet50_fpn(5, score_thresh=0.0), TD.fcos_resnet50_fpn(num_classes=5, score_thresh=0.0, **sized), x)
    else:
        _same_detections(M.ssd300_vgg16(5, normalize=False), TD.ssd300_vgg16(num_classes=5, **ident), torch.rand(2, 3, 300, 300))


def test_yolo_grid_and_decoding():
    from ferrotorch_b200.models import detection as M

    torch.manual_seed(7)
    net = M.yolo(4).eval()
    assert sorted(net.state_dict())[:2] == ["backbone.stage1.conv.weight", "backbone.stage2.conv.weight"] and "head.bias" in net.state_dict()
    grid = net(torch.rand(2, 3, 416, 416))
    assert grid.shape == (2, 3 * (5 + 4), 13, 13)
    det = net.decode(grid, [(30, 40), (80, 60), (150, 200)], (416, 416), conf_thresh=0.0, nms_thresh=0.5)
    for d in det:
        assert len(d["boxes"]) > 0 and d["boxes"].min() >= 0 and d["boxes"].max() <= 416
        assert (d["scores"][:-1] >= d["scores"][1:]).all() and set(d["labels"].tolist()) <= {0, 1, 2, 3}


def test_registry_prefers_own_models():
    from ferrotorch_b200 import vision as V
    from ferrotorch_b200.models import vision_zoo as Z

    assert isinstance(V.build("vgg16", num_classes=3), Z.VGG)
    assert isinstance(V.build("deeplabv3", num_classes=3), Z.SegmentationModel)
    from ferrotorch_b200.models import vision_families as M

    assert isinstance(V.build("efficientnet_b0", num_classes=3), M.EfficientNet)
    assert isinstance(V.build("swin_t", num_classes=3), M.SwinTransformer)
    assert isinstance(V.build("lraspp", num_classes=3), M.LRASPP)
    from ferrotorch_b200.models import detection as Dm

    assert isinstance(V.build("retinanet", num_classes=3), Dm.RetinaNet) and isinstance(V.build("yolo", num_classes=3), Dm.Yolo)


def test_every_vision_entry_of_the_hub_builds_with_its_listed_size():
    # the registry's parameter counts are the published sizes of these architectures
    from ferrotorch_b200 import hub
    from ferrotorch_b200 import vision as V

    seen = 0
    for info in hub.list_models():
        if "vision:build" not in info.builder:
            continue
        net = V.build(info.name)
        assert sum(p.numel() for p in net.parameters()) == info.num_parameters, info.name
        assert type(net).__module__.startswith("ferrotorch_b200."), "%s is not this package's own module" % info.name
        seen += 1
    assert seen >= 23


def test_every_name_of_the_reference_registry_builds_as_an_own_module():
    # the model names registered in ferrotorch-vision/src/models/registry.rs
    from ferrotorch_b200 import vision as V

    names = ["convnext_tiny", "deeplabv3_resnet50", "densenet121", "efficientnet_b0", "fasterrcnn_resnet50_fpn", "fcn_resnet50",
             "fcos_resnet50_fpn", "inception_v3", "keypointrcnn_resnet50_fpn", "lraspp_mobilenet_v3_large", "maskrcnn_resnet50_fpn",
             "mobilenet_v2", "mobilenet_v3_small", "resnet18", "resnet34", "resnet50", "retinanet_resnet50_fpn", "ssd300_vgg16",
             "swin_tiny", "unet", "vgg11", "vgg16", "vit_b_16", "yolo"]
    for n in names:
        net = V.build(n)
        assert type(net).__module__.startswith("ferrotorch_b200."), n
    assert set(names) <= set(V.available())
