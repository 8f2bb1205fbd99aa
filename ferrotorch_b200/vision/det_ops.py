"""Detection operators (NMS, RoI align, box coders, anchors): the implementation lives in
``ops/det_ops.py`` so that the model files can use it without importing this package; every name
is available here as well."""
from ..ops.det_ops import *  # noqa: F401,F403
from ..ops.det_ops import BBOX_XFORM_CLIP, _bilinear  # noqa: F401
