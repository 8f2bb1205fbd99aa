"""Model hub: a registry of named models, a checksummed weight cache, Hugging Face token lookup,
model search and snapshot download (ferrotorch-hub/src/{registry,cache,download,auth,discovery}.rs).

Everything that needs the network goes through :func:`_http_get`; where there is none, those calls
raise :class:`HubOffline` and the cache-only paths keep working (``load_pretrained`` on weights that
are already cached, ``hf_download_model`` on snapshots already in ``HF_HOME``)."""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import urllib.error
import urllib.parse
import urllib.request
from dataclasses import dataclass, field

from .utils.text import HfTransformerConfig, hf_cache_path  # noqa: F401


class HubOffline(ConnectionError):
    """The hub could not be reached."""


# --------------------------------------------------------------------------- registry
@dataclass(frozen=True)
class ModelInfo:
    name: str
    description: str
    builder: str                  # "module:callable" that constructs the architecture
    num_parameters: int
    weights_url: str = ""
    weights_sha256: str = ""
    format: str = "safetensors"   # or "pt"

    def build(self, **kw):
        mod, fn = self.builder.split(":")
        obj = __import__(mod, fromlist=["_"])
        for part in fn.split("."):
            obj = getattr(obj, part)
        return obj(**kw)


def _vision(name, desc, n):
    return ModelInfo(name, desc, "ferrotorch_b200.vision:build", n)


_MODELS = [
    _vision("resnet18", "ResNet-18, ImageNet-1K classifier", 11_689_512),
    _vision("resnet34", "ResNet-34, ImageNet-1K classifier", 21_797_672),
    _vision("resnet50", "ResNet-50, ImageNet-1K classifier", 25_557_032),
    _vision("vgg11", "VGG-11", 132_863_336), _vision("vgg16", "VGG-16", 138_357_544),
    _vision("vit_b_16", "ViT-B/16", 86_567_656), _vision("efficientnet_b0", "EfficientNet-B0", 5_288_548),
    _vision("swin_t", "Swin-T", 28_288_354), _vision("convnext_tiny", "ConvNeXt-T", 28_589_128),
    _vision("mobilenet_v2", "MobileNetV2", 3_504_872), _vision("mobilenet_v3_small", "MobileNetV3-Small", 2_542_856),
    _vision("densenet121", "DenseNet-121", 7_978_856), _vision("inception_v3", "Inception v3", 27_161_264),
    _vision("mobilenet_v3_large", "MobileNetV3-Large", 5_483_032),
    # detectors and segmenters: counts with trainable batch-norm affine parameters (checkpoints that freeze
    # them list 53 120 fewer) and without the auxiliary segmentation head
    _vision("fasterrcnn_resnet50_fpn", "Faster R-CNN, ResNet-50 FPN, 91 classes", 41_808_406),
    _vision("maskrcnn_resnet50_fpn", "Mask R-CNN, ResNet-50 FPN, 91 classes", 44_454_513),
    _vision("keypointrcnn_resnet50_fpn", "Keypoint R-CNN, ResNet-50 FPN, 17 keypoints", 59_190_378),
    _vision("retinanet_resnet50_fpn", "RetinaNet, ResNet-50 FPN, 91 classes", 34_068_119),
    _vision("fcos_resnet50_fpn", "FCOS, ResNet-50 FPN, 91 classes", 32_322_720),
    _vision("ssd300_vgg16", "SSD300, VGG-16, 91 classes", 35_641_826),
    _vision("fcn_resnet50", "FCN, dilated ResNet-50, 21 classes", 32_957_013),
    _vision("deeplabv3_resnet50", "DeepLabV3, dilated ResNet-50, 21 classes", 39_638_869),
    _vision("lraspp_mobilenet_v3_large", "LR-ASPP, MobileNetV3-Large, 21 classes", 3_221_538),
    ModelInfo("llama3-8b", "Llama-3-8B decoder", "ferrotorch_b200.models.llama:LlamaConfig.llama3_8b", 8_030_261_248),
    ModelInfo("llama3.3-70b-instruct", "Llama-3.3-70B-Instruct decoder",
              "ferrotorch_b200.models.llama:LlamaConfig.llama3_3_70b_instruct", 70_553_706_496),
    ModelInfo("all-MiniLM-L6-v2", "Sentence embeddings, 6-layer MiniLM", "ferrotorch_b200.models.pretrained:SentenceTransformer", 22_713_216),
    ModelInfo("whisper-tiny-encoder", "Whisper tiny audio encoder", "ferrotorch_b200.models.pretrained:WhisperEncoder", 8_208_384),
    ModelInfo("sd-v1-5-unet", "Stable Diffusion 1.5 UNet", "ferrotorch_b200.models.diffusion:UNet2DConditionModel", 859_520_964),
    ModelInfo("sd-v1-5-vae", "Stable Diffusion 1.5 VAE", "ferrotorch_b200.models.diffusion:AutoencoderKL", 83_653_863),
    ModelInfo("sd-v1-5-clip-text-encoder", "CLIP ViT-L/14 text tower", "ferrotorch_b200.models.diffusion:ClipTextEncoder", 123_060_480),
    ModelInfo("gcn-cora", "2-layer GCN", "ferrotorch_b200.models.pretrained:GcnNet", 23_063),
    ModelInfo("ppo-cartpole-v1", "SB3 PPO MlpPolicy for CartPole-v1", "ferrotorch_b200.models.pretrained:MlpPolicy", 9_155),
]
_BY_NAME = {m.name: m for m in _MODELS}


def list_models() -> list[ModelInfo]:
    return list(_MODELS)


def get_model_info(name: str) -> ModelInfo | None:
    return _BY_NAME.get(name)


# --------------------------------------------------------------------------- cache
def default_cache_dir() -> str:
    base = os.environ.get("FERROTORCH_CACHE") or os.path.join(
        os.environ.get("XDG_CACHE_HOME") or os.path.join(os.path.expanduser("~"), ".cache"), "ferrotorch")
    return os.path.join(base, "hub")


class HubCache:
    """Flat directory of weight files keyed by model name; names may not escape the directory."""

    def __init__(self, directory: str):
        self.dir = os.path.abspath(directory)

    @classmethod
    def with_default_dir(cls) -> "HubCache":
        return cls(default_cache_dir())

    def cache_dir(self) -> str:
        return self.dir

    def path(self, name: str) -> str:
        if not name or name in (".", "..") or "/" in name or "\\" in name or "\0" in name:
            raise ValueError("HubCache: %r is not a valid entry name" % (name,))
        return os.path.join(self.dir, name)

    def path_for_model(self, info: ModelInfo) -> str:
        return self.path("%s.%s" % (info.name, info.format))

    def has(self, name: str) -> bool:
        return os.path.isfile(self.path(name))

    def store(self, name: str, data: bytes) -> None:
        os.makedirs(self.dir, exist_ok=True)
        tmp = self.path(name) + ".part%d" % os.getpid()
        with open(tmp, "wb") as f:
            f.write(data)
        os.replace(tmp, self.path(name))

    def load(self, name: str) -> bytes:
        with open(self.path(name), "rb") as f:
            return f.read()

    def clear(self) -> None:
        if os.path.isdir(self.dir):
            shutil.rmtree(self.dir)


def sha256_hex(data: bytes) -> str:
    return hashlib.sha256(data).hexdigest()


# --------------------------------------------------------------------------- auth and transport
def hf_token() -> str | None:
    """``HF_TOKEN``, else the token file under ``HF_HOME``, else ``~/.cache/huggingface/token``
    (auth.rs:35-70); blank values count as absent."""
    t = os.environ.get("HF_TOKEN", "").strip()
    if t:
        return t
    cands = []
    if os.environ.get("HF_HOME"):
        cands.append(os.path.join(os.environ["HF_HOME"], "token"))
    cands.append(os.path.join(os.path.expanduser("~"), ".cache", "huggingface", "token"))
    for p in cands:
        try:
            with open(p) as f:
                t = f.read().strip()
            if t:
                return t
        except OSError:
            pass
    return None


def _http_get(url: str, timeout: float = 10.0) -> bytes:
    req = urllib.request.Request(url, headers={"User-Agent": "ferrotorch_b200"})
    tok = hf_token()
    if tok and urllib.parse.urlparse(url).hostname in ("huggingface.co", "hf.co"):
        req.add_header("Authorization", "Bearer " + tok)
    try:
        with urllib.request.urlopen(req, timeout=timeout) as r:
            return r.read()
    except (urllib.error.URLError, OSError, TimeoutError) as e:
        raise HubOffline("cannot reach %s: %s" % (url, e))


# --------------------------------------------------------------------------- weights
def download_weights(info: ModelInfo, cache: HubCache | None = None) -> str:
    """Path of the model's weight file in the cache, downloading it first if needed; the file's
    SHA-256 must equal ``info.weights_sha256`` when one is recorded (download.rs:40)."""
    cache = cache or HubCache.with_default_dir()
    name = "%s.%s" % (info.name, info.format)
    if not cache.has(name):
        if not info.weights_url:
            raise FileNotFoundError("no weights are published for %r and none are cached under %s" % (info.name, cache.cache_dir()))
        cache.store(name, _http_get(info.weights_url, timeout=60.0))
    if info.weights_sha256:
        got = sha256_hex(cache.load(name))
        if got != info.weights_sha256.lower():
            os.remove(cache.path(name))
            raise ValueError("checksum mismatch for %s: expected %s, got %s (the cached file was removed)"
                             % (info.name, info.weights_sha256, got))
    return cache.path(name)


def load_pretrained(name: str, cache: HubCache | None = None) -> dict:
    """State dict of a registered model from the cache (downloaded when missing and reachable)."""
    info = get_model_info(name)
    if info is None:
        raise KeyError("unknown model %r; known: %s" % (name, ", ".join(sorted(_BY_NAME))))
    path = download_weights(info, cache)
    if info.format == "safetensors":
        from .serialize.state import load_safetensors

        return load_safetensors(path)
    from .serialize.state import load_pytorch_state_dict

    return load_pytorch_state_dict(path)


def hf_download_model(repo_id: str, files: list[str] | None = None) -> str:
    """Directory holding ``repo_id``'s files: the newest snapshot in the local HF cache when there
    is one, else the listed ``files`` (default ``config.json``, ``model.safetensors``) fetched from
    the hub into that cache layout (download.rs:438)."""
    snaps = os.path.join(hf_cache_path(repo_id), "snapshots")
    if os.path.isdir(snaps) and os.listdir(snaps):
        return os.path.join(snaps, sorted(os.listdir(snaps))[-1])
    dest = os.path.join(snaps, "main")
    blobs = {f: _http_get("https://huggingface.co/%s/resolve/main/%s" % (repo_id, f), timeout=120.0)
             for f in (files or ["config.json", "model.safetensors"])}
    os.makedirs(dest, exist_ok=True)
    for f, data in blobs.items():
        with open(os.path.join(dest, f), "wb") as out:
            out.write(data)
    return dest


# --------------------------------------------------------------------------- discovery
@dataclass
class SearchQuery:
    search: str | None = None
    pipeline_tag: str | None = None
    library: str | None = None
    limit: int | None = None
    sort: str | None = None

    def with_search(self, s: str) -> "SearchQuery":
        self.search = s
        return self

    def with_pipeline_tag(self, t: str) -> "SearchQuery":
        self.pipeline_tag = t
        return self

    def with_library(self, lib: str) -> "SearchQuery":
        self.library = lib
        return self

    def with_limit(self, n: int) -> "SearchQuery":
        self.limit = max(1, min(int(n), 1000))
        return self

    def with_sort(self, key: str) -> "SearchQuery":
        self.sort = key
        return self

    def to_query_string(self) -> str:
        pairs = [("search", self.search), ("pipeline_tag", self.pipeline_tag), ("library", self.library),
                 ("limit", self.limit), ("sort", self.sort)]
        q = [(k, str(v)) for k, v in pairs if v is not None]
        if self.sort:
            q.append(("direction", "-1"))
        return urllib.parse.urlencode(q)


@dataclass
class HfModelSummary:
    id: str
    author: str | None = None
    downloads: int = 0
    likes: int = 0
    pipeline_tag: str | None = None
    tags: list = field(default_factory=list)

    @classmethod
    def from_json(cls, d: dict) -> "HfModelSummary":
        mid = d.get("id") or d.get("modelId") or ""
        return cls(mid, d.get("author") or (mid.split("/")[0] if "/" in mid else None), int(d.get("downloads") or 0),
                   int(d.get("likes") or 0), d.get("pipeline_tag"), list(d.get("tags") or []))


def search_models(query: SearchQuery) -> list[HfModelSummary]:
    data = json.loads(_http_get("https://huggingface.co/api/models?" + query.to_query_string()))
    return [HfModelSummary.from_json(d) for d in data]


def get_model(repo_id: str) -> dict:
    if not repo_id.strip():
        raise ValueError("get_model: empty repository id")
    return json.loads(_http_get("https://huggingface.co/api/models/" + urllib.parse.quote(repo_id, safe="/")))


# --------------------------------------------------------------------------- the reference's remaining type names
import enum as _enum  # noqa: E402


class WeightsFormat(str, _enum.Enum):
    """``ModelInfo.format`` values (registry.rs:21)."""
    SafeTensors = "safetensors"
    FerrotorchStateDict = "ftsd"
    PyTorch = "pt"

    def __str__(self) -> str:
        return self.value

    @property
    def extension(self) -> str:
        return {"safetensors": "safetensors", "ftsd": "fts", "pt": "pt"}[self.value]


class EntryKind(_enum.Enum):
    """A registry entry is a real model (positive parameter count) or a test fixture (registry.rs:38)."""
    Model = "model"
    Fixture = "fixture"

    @classmethod
    def of(cls, info: "ModelInfo") -> "EntryKind":
        return cls.Model if info.num_parameters > 0 else cls.Fixture


@dataclass
class HfRepoFile:
    rfilename: str


@dataclass
class HfModelInfo:
    """One repository as the hub's ``/api/models/<id>`` describes it (discovery.rs:99)."""
    model_id: str
    author: str | None = None
    downloads: int | None = None
    likes: int | None = None
    tags: list = field(default_factory=list)
    pipeline_tag: str | None = None
    siblings: list = field(default_factory=list)

    @classmethod
    def from_json(cls, d: dict) -> "HfModelInfo":
        mid = d.get("modelId") or d.get("id") or ""
        return cls(mid, d.get("author") or (mid.split("/")[0] if "/" in mid else None), d.get("downloads"), d.get("likes"),
                   list(d.get("tags") or []), d.get("pipeline_tag"),
                   [HfRepoFile(s["rfilename"]) for s in d.get("siblings") or [] if "rfilename" in s])

    def files(self) -> list:
        return [s.rfilename for s in self.siblings]


def get_model_details(repo_id: str) -> HfModelInfo:
    """:func:`get_model` parsed into :class:`HfModelInfo`."""
    return HfModelInfo.from_json(get_model(repo_id))


def with_auth(request: "urllib.request.Request") -> "urllib.request.Request":
    """Add ``Authorization: Bearer <token>`` when a hub token is configured (auth.rs:73); the
    request is returned unchanged otherwise, which is what public repositories expect."""
    tok = hf_token()
    if tok:
        request.add_header("Authorization", "Bearer " + tok)
    return request
