"""Hub: registry, checksummed cache, token lookup, query strings; network calls fail as HubOffline."""
import os

import pytest
import torch

from ferrotorch_b200 import hub as H


def test_registry_names_build_real_architectures():
    names = {m.name for m in H.list_models()}
    assert {"resnet18", "resnet50", "vit_b_16", "all-MiniLM-L6-v2", "whisper-tiny-encoder", "sd-v1-5-unet", "gcn-cora",
            "ppo-cartpole-v1"} <= names
    assert H.get_model_info("nope") is None
    for name, kw in [("ppo-cartpole-v1", {}), ("gcn-cora", {"in_features": 1433, "hidden": 16, "num_classes": 7}),
                     ("resnet18", {"name": "resnet18"})]:
        info = H.get_model_info(name)
        model = info.build(**kw)
        assert sum(p.numel() for p in model.parameters()) == info.num_parameters, name
    with torch.device("meta"):
        for name in ("all-MiniLM-L6-v2", "whisper-tiny-encoder", "sd-v1-5-clip-text-encoder"):
            info = H.get_model_info(name)
            assert sum(p.numel() for p in info.build().parameters()) == info.num_parameters, name
    assert H.get_model_info("llama3-8b").build().num_parameters() == H.get_model_info("llama3-8b").num_parameters


def test_cache_checksums_and_pretrained_loading(tmp_path):
    from ferrotorch_b200.serialize.state import save_safetensors

    cache = H.HubCache(str(tmp_path / "hub"))
    assert not cache.has("x.bin")
    cache.store("x.bin", b"abc")
    assert cache.has("x.bin") and cache.load("x.bin") == b"abc" and cache.path("x.bin").startswith(cache.cache_dir())
    for bad in ("../evil", "a/b", "", ".."):
        with pytest.raises(ValueError):
            cache.path(bad)
    sd = {"w": torch.arange(4.0)}
    save_safetensors(sd, str(tmp_path / "m.safetensors"))
    blob = (tmp_path / "m.safetensors").read_bytes()
    info = H.ModelInfo("toy", "toy", "torch.nn:Identity", 4, weights_sha256=H.sha256_hex(blob))
    cache.store("toy.safetensors", blob)
    assert H.download_weights(info, cache) == cache.path_for_model(info)
    H._BY_NAME["toy"] = info
    try:
        assert torch.equal(H.load_pretrained("toy", cache)["w"], sd["w"])
        cache.store("toy.safetensors", blob + b"x")                        # a corrupted file is rejected and removed
        with pytest.raises(ValueError, match="checksum mismatch"):
            H.load_pretrained("toy", cache)
        assert not cache.has("toy.safetensors")
        with pytest.raises(FileNotFoundError):
            H.load_pretrained("toy", cache)                                # nothing cached, nothing published
    finally:
        del H._BY_NAME["toy"]
    with pytest.raises(KeyError):
        H.load_pretrained("unknown-model", cache)
    cache.clear()
    assert not os.path.isdir(cache.cache_dir())


def test_token_lookup_order(tmp_path, monkeypatch):
    monkeypatch.setenv("HOME", str(tmp_path / "home"))
    monkeypatch.delenv("HF_TOKEN", raising=False)
    monkeypatch.delenv("HF_HOME", raising=False)
    assert H.hf_token() is None
    d = tmp_path / "home" / ".cache" / "huggingface"
    d.mkdir(parents=True)
    (d / "token").write_text(" home-token \n")
    assert H.hf_token() == "home-token"
    hf = tmp_path / "hfhome"
    hf.mkdir()
    (hf / "token").write_text("hfhome-token")
    monkeypatch.setenv("HF_HOME", str(hf))
    assert H.hf_token() == "hfhome-token"
    monkeypatch.setenv("HF_TOKEN", "   ")
    assert H.hf_token() == "hfhome-token"                                  # blank counts as absent
    monkeypatch.setenv("HF_TOKEN", "env-token")
    assert H.hf_token() == "env-token"


def test_queries_and_offline_errors(tmp_path, monkeypatch):
    q = H.SearchQuery().with_search("llama 3").with_pipeline_tag("text-generation").with_library("safetensors").with_limit(5000).with_sort("downloads")
    assert q.to_query_string() == "search=llama+3&pipeline_tag=text-generation&library=safetensors&limit=1000&sort=downloads&direction=-1"
    assert H.SearchQuery().to_query_string() == ""
    s = H.HfModelSummary.from_json({"modelId": "meta-llama/Llama-3-8B", "downloads": 7, "tags": ["a"]})
    assert (s.id, s.author, s.downloads, s.likes, s.tags) == ("meta-llama/Llama-3-8B", "meta-llama", 7, 0, ["a"])

    def refuse(*a, **k):
        raise OSError("network is unreachable")

    monkeypatch.setattr(H.urllib.request, "urlopen", refuse)
    with pytest.raises(H.HubOffline):
        H.search_models(q)
    with pytest.raises(H.HubOffline):
        H.get_model("meta-llama/Llama-3-8B")
    with pytest.raises(ValueError):
        H.get_model("  ")
    monkeypatch.setenv("HF_HOME", str(tmp_path / "hf"))
    with pytest.raises(H.HubOffline):
        H.hf_download_model("org/model")
    snap = tmp_path / "hf" / "hub" / "models--org--model" / "snapshots" / "abc"
    snap.mkdir(parents=True)
    (snap / "config.json").write_text("{}")
    assert H.hf_download_model("org/model") == str(snap)                    # a cached snapshot needs no network
    assert isinstance(H.HubOffline("x"), ConnectionError)


def test_hub_reference_type_names(monkeypatch):
    import urllib.request

    from ferrotorch_b200 import hub as H

    info = H.HfModelInfo.from_json({"modelId": "org/m", "downloads": 5, "tags": ["llama"],
                                    "siblings": [{"rfilename": "config.json"}, {"rfilename": "model.safetensors"}]})
    assert info.model_id == "org/m" and info.author == "org" and info.files() == ["config.json", "model.safetensors"]
    assert isinstance(info.siblings[0], H.HfRepoFile) and info.likes is None
    assert H.WeightsFormat.SafeTensors == "safetensors" and H.WeightsFormat.FerrotorchStateDict.extension == "fts"
    assert all(H.EntryKind.of(m) is H.EntryKind.Model for m in H.list_models())
    monkeypatch.setenv("HF_TOKEN", "abc")
    req = H.with_auth(urllib.request.Request("https://huggingface.co/api/models/x"))
    assert req.get_header("Authorization") == "Bearer abc"
    monkeypatch.delenv("HF_TOKEN")
    monkeypatch.setenv("HF_HOME", "/nonexistent-dir-for-test")
    monkeypatch.delenv("HUGGING_FACE_HUB_TOKEN", raising=False)
    req = H.with_auth(urllib.request.Request("https://huggingface.co/api/models/x"))
    assert req.get_header("Authorization") is None
