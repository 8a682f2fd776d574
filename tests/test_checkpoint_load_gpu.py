"""litnice_b200_load_checkpoint: the direct reader of version-6 checkpoint files
(checkpoint.cpp:588-652). A loaded file must behave exactly like the same arena
handed over from host memory, and the loader must refuse what the reference
refuses: a short file, another model's dimensions or alignment
(checkpoint.cpp:609-628), non-finite parameters (:176-205). Also the session
state rules around forward / run and resumed runs.
"""
import struct

import numpy as np
import pytest

from litnicelm_b200 import formats
from litnicelm_b200.plugin import NativeError, Session

pytestmark = pytest.mark.gpu

D = formats.ModelDims(2, 2, 64, 256, 96, 48)


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    arena = formats.make_param_arena(D, 77, bias_std=0.02, ln_std=0.1)
    path = str(tmp_path_factory.mktemp("ckpt") / "m.ckpt")
    formats.write_checkpoint(path, D, arena)
    return arena, path


def test_checkpoint_round_trip_equals_load_params(model):
    arena, path = model
    ids = formats.zipf_prompt(D.vocab, 20, 5)
    with Session(D, 1) as a, Session(D, 1) as b:
        a.load_params(arena)
        b.load_checkpoint(path)
        assert np.array_equal(a.forward(ids, all_rows=True), b.forward(ids, all_rows=True))
        assert np.array_equal(a.generate(ids, 12), b.generate(ids, 12))
    d2, arena2 = formats.read_checkpoint(path)
    assert d2 == D and np.array_equal(arena2, arena)


def _expect_refusal(path, pattern, dims=D):
    with Session(dims, 1) as s:
        with pytest.raises(NativeError, match=pattern):
            s.load_checkpoint(path)
        # a refused load leaves the session without parameters
        with pytest.raises(NativeError, match="no parameters loaded"):
            s.forward(np.zeros(4, np.int32))


def test_truncated_files_are_refused(model, tmp_path):
    _, path = model
    raw = open(path, "rb").read()
    short_header = str(tmp_path / "h.ckpt")
    open(short_header, "wb").write(raw[:100])
    _expect_refusal(short_header, "truncated v6 header")
    short_payload = str(tmp_path / "p.ckpt")
    open(short_payload, "wb").write(raw[:formats.CKPT_HEADER_BYTES + 1000])
    _expect_refusal(short_payload, "could not read parameter arena")
    _expect_refusal(str(tmp_path / "absent.ckpt"), "cannot open checkpoint")


def test_wrong_magic_dimensions_and_alignment_are_refused(model, tmp_path):
    _, path = model
    raw = bytearray(open(path, "rb").read(formats.CKPT_HEADER_BYTES + 4096))
    bad_magic = str(tmp_path / "magic.ckpt")
    open(bad_magic, "wb").write(struct.pack("<I", 0x12345678) + bytes(raw[4:]))
    _expect_refusal(bad_magic, "not a version-6")
    # the same file read by a session of another shape / alignment
    _expect_refusal(path, "incompatible checkpoint", formats.ModelDims(2, 2, 64, 256, 96, 64))
    _expect_refusal(path, "incompatible checkpoint", formats.ModelDims(3, 2, 64, 256, 96, 48))
    _expect_refusal(path, "incompatible checkpoint", formats.ModelDims(2, 2, 64, 256, 96, 48, alignment=128))


@pytest.mark.parametrize("poison", [np.nan, np.inf, -np.inf])
def test_non_finite_parameters_are_refused(model, tmp_path, poison):
    arena, _ = model
    bad = arena.copy()
    lay = formats.ParamLayout.build(D)
    lay.view(bad, "layer1.ffn_w2")[3, 5] = poison
    path = str(tmp_path / "nan.ckpt")
    formats.write_checkpoint(path, D, bad)
    _expect_refusal(path, "non-finite")


def test_forward_between_upload_and_run_demands_a_fresh_upload(model):
    """forward and inspect overwrite the token ids of an uploaded prompt batch, so a
    run that follows them without a new upload is refused instead of decoding stale ids."""
    arena, _ = model
    ids = formats.zipf_prompt(D.vocab, 10, 6)
    with Session(D, 1) as s:
        s.load_params(arena)
        want = s.generate(ids, 8)
        s.upload_prompts(ids)
        s.forward(formats.zipf_prompt(D.vocab, 14, 7))
        with pytest.raises(NativeError, match="no prompts uploaded"):
            s.run(8)
        s.upload_prompts(ids)
        s.inspect(formats.zipf_prompt(D.vocab, 14, 8))
        with pytest.raises(NativeError, match="no prompts uploaded"):
            s.run(8)
        s.upload_prompts(ids)
        assert s.run(8) == 8
        assert np.array_equal(s.download_tokens(8), want)


def test_resumed_run_keeps_tokens_and_step_logits(model):
    arena, _ = model
    ids = formats.zipf_prompt(D.vocab, 10, 9)
    with Session(D, 1) as s:
        s.load_params(arena)
        s.keep_step_logits(True)
        whole = s.generate(ids, 12)
        whole_logits = s.read_step_logits(12, 1)
        s.upload_prompts(ids)
        assert s.run(5) == 5
        assert s.run(7) == 12            # resumes: 5 tokens already there
        parts = s.download_tokens(12)
        parts_logits = s.read_step_logits(12, 1)
    assert np.array_equal(parts, whole)
    assert np.array_equal(parts_logits, whole_logits)


def test_read_file2device_of_the_plugin_table(tmp_path):
    """read_file2device (backend_plugin_api.hpp:158-160, CPU semantics device_backend.cpp:1752-1775):
    a byte range of a file lands in device memory; ranges larger than one staging piece and
    ranges that run past the end of the file are covered."""
    from litnicelm_b200.plugin import Backend
    data = np.random.default_rng(3).integers(0, 256, size=(40 << 20) + 12345, dtype=np.uint8)
    path = str(tmp_path / "blob.bin")
    data.tofile(path)
    with Backend() as be:
        assert be.call("is_file2device_read_supported") == 1
        for offset, size in ((0, 4096), (777, (33 << 20) + 5), (len(data) - 100, 100)):
            ptr = be.alloc(size + 64)
            be.api.read_file2device(be.h, path.encode(), ptr, size, offset)
            assert np.array_equal(be.download(ptr, size), data[offset:offset + size])
        ptr = be.alloc(4096)
        be.api.read_file2device(be.h, path.encode(), ptr, 0, 0)       # size 0: nothing to do
    from training_util import child_raises
    child_raises(f"""
ptr = be.alloc(4096)
be.api.read_file2device(be.h, {path!r}.encode(), ptr, 4096, {len(data) - 10})
""", "read_file2device: short read")
    child_raises(f"""
ptr = be.alloc(4096)
be.api.read_file2device(be.h, {str(tmp_path / "absent")!r}.encode(), ptr, 16, 0)
""", "read_file2device: failed to open")
