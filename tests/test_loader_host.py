"""Host side of the checkpoint loader (no GPU): header parsing, the manifest checks that
must reject a bad checkpoint before any device memory is touched (upstream contract:
src/weight_loader.rs:9-16 — duplicate, missing, unexpected, wrong dtype, wrong shape,
overlapping or out-of-range tensors), and the sizing of the device blocks."""
import json
import os

import numpy as np
import pytest

from helpers import make_moe_inputs, moe_checkpoint_tensors, write_raw_safetensors, write_safetensors

PREFIX = "model.language_model.layers.3.mlp."
H, I, E, S = 128, 64, 6, 64


@pytest.fixture(scope="module")
def ops():
    from qs3_b200 import ops as m
    return m


@pytest.fixture(scope="module")
def loader():
    from qs3_b200 import loader as m
    return m


@pytest.fixture(scope="module")
def ctx(ops):
    return ops.Context(device=-1)   # host-only context: nothing below makes a CUDA call


@pytest.fixture(scope="module")
def inputs():
    return make_moe_inputs(5, 4, H, E, I, S)


def _open_error(ops, loader, ctx, directory):
    with pytest.raises(ops.Qs3Error) as err:
        loader.Checkpoint(ctx, str(directory))
    assert err.value.status == ops.capi.STATUS_INVALID_ARGUMENT
    return str(err.value)


def _bf16_dir(tmp_path, inputs, **kw):
    tensors, _ = moe_checkpoint_tensors(PREFIX, inputs, nvfp4=False, **kw)
    write_safetensors(tmp_path / "model.safetensors", tensors)
    return tensors


def test_headers_index_and_config_are_parsed(tmp_path, ops, loader, ctx, inputs):
    tensors, _ = moe_checkpoint_tensors(PREFIX, inputs, nvfp4=False)
    names = list(tensors)
    first = {n: tensors[n] for n in names[:2]}
    second = {n: tensors[n] for n in names[2:]}
    second["model.visual.patch_embed.weight"] = ("F16", (2, 3), np.arange(6, dtype=np.float16))
    second["odd \"name\" é"] = ("I64", (2,), np.array([7, -9], np.int64))
    write_safetensors(tmp_path / "model-00001-of-00002.safetensors", first, metadata={"format": "pt"})
    write_safetensors(tmp_path / "model-00002-of-00002.safetensors", second)
    index = {"metadata": {"total_size": 1}, "weight_map": {}}
    for n in first:
        index["weight_map"][n] = "model-00001-of-00002.safetensors"
    for n in second:
        index["weight_map"][n] = "model-00002-of-00002.safetensors"
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    (tmp_path / "config.json").write_text(json.dumps({
        "architectures": ["X"], "text_config": {
            "hidden_size": H, "moe_intermediate_size": I, "num_experts": E, "num_experts_per_tok": 2,
            "shared_expert_intermediate_size": S, "num_hidden_layers": 40, "norm_topk_prob": True,
            "rms_norm_eps": 1e-6, "rope_theta": 1e7, "nested": {"a": [1, 2.5, None, False]}}}))
    ck = loader.Checkpoint(ctx, str(tmp_path))
    infos = ck.tensors()
    assert [t.name for t in infos] == sorted(list(first) + list(second))
    for t in infos:
        dtype, shape, data = {**first, **second}[t.name]
        assert (t.dtype, t.shape) == (dtype, tuple(shape))
        assert np.array_equal(ck.read_host(t.name), np.asarray(data).reshape(shape))
        assert os.path.basename(t.file) == index["weight_map"][t.name]
    gu = ck.find(PREFIX + "experts.gate_up_proj")
    assert gu.shape == (E, 2 * I, H) and gu.nbytes == E * 2 * I * H * 2
    cfg = ck.moe_config()
    assert (cfg.hidden_size, cfg.intermediate_size, cfg.num_experts, cfg.top_k, cfg.shared_intermediate_size,
            cfg.num_layers, cfg.renormalize) == (H, I, E, 2, S, 40, 1)
    assert cfg.rms_norm_eps == pytest.approx(1e-6)
    with pytest.raises(ops.Qs3Error, match="missing tensor"):
        ck.find("nope")


def test_directory_without_index_uses_every_shard(tmp_path, loader, ctx):
    write_safetensors(tmp_path / "b.safetensors", {"y": ("U8", (3,), np.array([1, 2, 3], np.uint8))})
    write_safetensors(tmp_path / "a.safetensors", {"x": ("F32", (), np.float32(2.5)),
                                                   "empty": ("F32", (0, 4), np.zeros((0, 4), np.float32))})
    (tmp_path / "notes.txt").write_text("not a shard")
    ck = loader.Checkpoint(ctx, str(tmp_path) + "/")
    assert [t.name for t in ck.tensors()] == ["empty", "x", "y"]
    assert ck.read_host("x") == np.float32(2.5)
    assert ck.read_host("empty").shape == (0, 4)
    with pytest.raises(Exception, match="config.json"):
        ck.moe_config()


def _entry(dtype, shape, begin, end):
    return {"dtype": dtype, "shape": shape, "data_offsets": [begin, end]}


@pytest.mark.parametrize("header,data,fragment", [
    ({"a": _entry("F32", [2], 0, 8), "b": _entry("F32", [2], 4, 12)}, 12, "overlap"),
    ({"a": _entry("F32", [4], 0, 16)}, 12, "out of range"),
    ({"a": _entry("F32", [3], 0, 8)}, 8, "shape and dtype need 12"),
    ({"a": _entry("F4", [2], 0, 1)}, 1, "unknown dtype"),
    ({"a": _entry("F32", [-1], 0, 4)}, 4, "malformed shape"),
    ({"a": _entry("F32", [1.5], 0, 4)}, 4, "malformed shape"),
    ({"a": _entry("F32", [1], 4, 0)}, 4, "malformed data_offsets"),
    ({"a": {"dtype": "F32", "shape": [1]}}, 4, "malformed entry"),
    ({"a": _entry("F32", [1] * 9, 0, 4)}, 4, "more than 8 dimensions"),
    ({"a": _entry("U8", [1 << 40, 1 << 40], 0, 4)}, 4, "overflows"),
])
def test_bad_shard_headers_are_rejected(tmp_path, ops, loader, ctx, header, data, fragment):
    write_raw_safetensors(tmp_path / "model.safetensors", json.dumps(header), b"\0" * data)
    assert fragment in _open_error(ops, loader, ctx, tmp_path)


def test_malformed_files_are_rejected(tmp_path, ops, loader, ctx):
    assert "no safetensors shard" in _open_error(ops, loader, ctx, tmp_path)
    assert "cannot open checkpoint directory" in _open_error(ops, loader, ctx, tmp_path / "absent")
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x01\x02")
    assert "shorter than a safetensors header" in _open_error(ops, loader, ctx, tmp_path)
    p.write_bytes((1 << 40).to_bytes(8, "little") + b"{}")
    assert "outside the file" in _open_error(ops, loader, ctx, tmp_path)
    write_raw_safetensors(p, '{"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]', b"\0" * 4)
    assert "not a JSON object" in _open_error(ops, loader, ctx, tmp_path)
    write_raw_safetensors(p, "[1, 2]")
    assert "not a JSON object" in _open_error(ops, loader, ctx, tmp_path)
    # the same name twice in one header: most JSON readers keep the last one silently
    write_raw_safetensors(p, '{"a": {"dtype":"U8","shape":[1],"data_offsets":[0,1]},'
                             ' "a": {"dtype":"U8","shape":[1],"data_offsets":[1,2]}}', b"\0\0")
    assert "duplicate tensor a" in _open_error(ops, loader, ctx, tmp_path)


def test_duplicates_and_index_mismatches_are_rejected(tmp_path, ops, loader, ctx):
    one = {"x": ("U8", (2,), np.array([1, 2], np.uint8))}
    write_safetensors(tmp_path / "a.safetensors", one)
    write_safetensors(tmp_path / "b.safetensors", {**one, "y": ("U8", (1,), np.array([3], np.uint8))})
    assert "duplicate tensor x" in _open_error(ops, loader, ctx, tmp_path)
    index = tmp_path / "model.safetensors.index.json"
    index.write_text(json.dumps({"weight_map": {"x": "a.safetensors", "y": "a.safetensors"}}))
    assert "missing tensor y" in _open_error(ops, loader, ctx, tmp_path)       # y is in b, the index says a
    index.write_text(json.dumps({"weight_map": {"x": "a.safetensors", "z": "a.safetensors"}}))
    assert "missing tensor z" in _open_error(ops, loader, ctx, tmp_path)
    index.write_text(json.dumps({"weight_map": {"y": "b.safetensors"}}))
    assert "unexpected tensor x" in _open_error(ops, loader, ctx, tmp_path)    # b also holds x, not indexed
    index.write_text(json.dumps({"weight_map": {"x": "../a.safetensors"}}))
    assert "not a plain file name" in _open_error(ops, loader, ctx, tmp_path)
    index.write_text(json.dumps({"metadata": {}}))
    assert "no weight_map" in _open_error(ops, loader, ctx, tmp_path)
    index.write_text('{"weight_map": {"x": "a.safetensors", "x": "a.safetensors"}}')
    assert "duplicate tensor x" in _open_error(ops, loader, ctx, tmp_path)


def _aligned(n):
    return (n + 255) // 256 * 256


def test_bf16_layer_manifest_and_sizes(tmp_path, ops, loader, ctx, inputs):
    capi = ops.capi
    _bf16_dir(tmp_path, inputs)
    ck = loader.Checkpoint(ctx, str(tmp_path))
    dims = dict(hidden=H, inter=I, experts=E, shared_inter=S)
    weight, scratch = ck.layer_bytes(PREFIX, **dims)
    want = sum(_aligned(n) for n in (E * H * 2, E * 2 * I * H * 2, E * H * I * 2, 2 * S * H * 2, H * S * 2, H * 2))
    assert (weight, scratch) == (want, 0)          # file layout = kernel layout: nothing is staged
    # a rank that holds experts 2..3 only
    weight_local, _ = ck.layer_bytes(PREFIX, local=(2, 2), **dims)
    assert weight - weight_local == _aligned(E * 2 * I * H * 2) - _aligned(2 * 2 * I * H * 2) \
        + _aligned(E * H * I * 2) - _aligned(2 * H * I * 2)
    # quantising at load time stages bf16 chunks (two halves of min(E, 8) experts) and the shared expert
    weight_q, scratch_q = ck.layer_bytes(PREFIX, backend=capi.MOE_BACKEND_NVFP4, **dims)
    assert weight_q < weight
    assert scratch_q >= 2 * E * (2 * I * H + H * I) * 2 + (2 * S * H + H * S) * 2
    for bad, fragment in [
        (dict(dims, hidden=H * 2), "has shape"),
        (dict(dims, experts=E + 1), "has shape"),
        (dict(dims, shared_inter=0), "unexpected tensor " + PREFIX + "shared_expert"),
        (dict(dims, local=(4, 4)), "local expert range"),
        (dict(dims, expert_order=[0, 1, 2, 3, 4, 4]), "not a permutation"),
        (dict(dims, fmt=capi.CHECKPOINT_EXPERTS_NVFP4_SPLIT, backend=capi.MOE_BACKEND_NVFP4), "missing tensor"),
        (dict(dims, backend=capi.MOE_BACKEND_FP8_BLOCKSCALE), "BF16 or NVFP4 layouts only"),
    ]:
        with pytest.raises(ops.Qs3Error, match=fragment):
            ck.layer_bytes(PREFIX, **bad)
    with pytest.raises(ops.Qs3Error, match="missing tensor model.layers.0.mlp.gate.weight"):
        ck.layer_bytes("model.layers.0.mlp.", **dims)


def test_transposed_fused_tensors_are_recognised(tmp_path, loader, ctx, inputs):
    _bf16_dir(tmp_path, inputs, transposed=True)
    ck = loader.Checkpoint(ctx, str(tmp_path))
    dims = dict(hidden=H, inter=I, experts=E, shared_inter=S)
    # hidden == 2 * intermediate here: [E, 2I, H] and [E, H, 2I] are the same shape, the caller decides
    _, scratch = ck.layer_bytes(PREFIX, fused_transposed=True, **dims)
    assert scratch == 2 * E * (2 * I * H + H * I) * 2     # both staged, then transposed on the device
    _, scratch = ck.layer_bytes(PREFIX, **dims)
    assert scratch == 2 * E * H * I * 2                   # down_proj is unambiguous: [E, I, H]


def test_nvfp4_layer_manifest(tmp_path, ops, loader, ctx, inputs):
    capi = ops.capi
    tensors, _ = moe_checkpoint_tensors(PREFIX, inputs, nvfp4=True)
    write_safetensors(tmp_path / "model.safetensors", tensors)
    ck = loader.Checkpoint(ctx, str(tmp_path))
    kw = dict(hidden=H, inter=I, experts=E, shared_inter=S, fmt=capi.CHECKPOINT_EXPERTS_NVFP4_SPLIT,
              backend=capi.MOE_BACKEND_NVFP4)
    weight, scratch = ck.layer_bytes(PREFIX, **kw)
    tiled = lambda rows, k: ops.nvfp4_tiled_scale_bytes(rows, k)
    want = sum(_aligned(n) for n in (
        E * H * 2, E * 2 * I * H // 2, E * H * I // 2, E * tiled(2 * I, H), E * tiled(H, I), 2 * E * 4, E * 4,
        2 * S * H // 2, H * S // 2, tiled(2 * S, H), tiled(H, S), 8, 4, H * 2))
    assert weight == want
    assert scratch >= 2 * E * (2 * I * H // 16 + H * I // 16)
    with pytest.raises(ops.Qs3Error, match="cannot be loaded into a BF16 plan"):
        ck.layer_bytes(PREFIX, **dict(kw, backend=capi.MOE_BACKEND_FUSED_BF16))

    def broken(change):
        t = dict(tensors)
        change(t)
        d = tmp_path / f"broken{len(os.listdir(tmp_path))}"
        d.mkdir()
        write_safetensors(d / "model.safetensors", t)
        return loader.Checkpoint(ctx, str(d))

    stem = PREFIX + "experts.4.up_proj"
    cases = [
        (lambda t: t.pop(stem + ".weight_scale_2"), "missing tensor " + stem + ".weight_scale_2"),
        (lambda t: t.__setitem__(stem + ".weight_scale", ("U8",) + t[stem + ".weight_scale"][1:]),
         "has dtype U8, expected F8_E4M3"),
        (lambda t: t.__setitem__(stem + ".weight", ("U8", (I // 2, H), t[stem + ".weight"][2])), "has shape"),
        (lambda t: t.__setitem__(stem + ".input_scale", ("F32", (2,), np.zeros(2, np.float32))), "expected a scalar"),
        (lambda t: t.__setitem__(PREFIX + "experts.6.gate_proj.weight", t[stem + ".weight"]), "unexpected tensor"),
        (lambda t: t.__setitem__(PREFIX + "gate.bias", ("F32", (E,), np.zeros(E, np.float32))), "unexpected tensor"),
    ]
    for change, fragment in cases:
        with pytest.raises(ops.Qs3Error, match=fragment):
            broken(change).layer_bytes(PREFIX, **kw)


def test_load_refuses_missing_device_blocks(tmp_path, ops, loader, ctx, inputs):
    """The load entry validates the manifest and its buffers before the first CUDA call, so
    these rejections are reachable without a GPU."""
    import ctypes as C
    _bf16_dir(tmp_path, inputs)
    ck = loader.Checkpoint(ctx, str(tmp_path))
    d, _keep = ck._layer_desc(PREFIX, H, I, E, S, 0, ops.capi.MOE_BACKEND_FUSED_BF16, None, None, False)
    out = ops.capi.MoeLayerWeights()
    lib = ops.capi.load()
    status = lib.qs3_checkpoint_load_moe_layer(ctx.handle, ck.handle, C.byref(d), None, 0, None, 0, C.byref(out))
    assert status == ops.capi.STATUS_INVALID_ARGUMENT
    assert b"weight block" in ctx.last_error().message
    d.hidden_size = H + 8
    status = lib.qs3_checkpoint_load_moe_layer(ctx.handle, ck.handle, C.byref(d), None, 0, None, 0, C.byref(out))
    assert status == ops.capi.STATUS_INVALID_ARGUMENT
    assert b"has shape" in ctx.last_error().message
