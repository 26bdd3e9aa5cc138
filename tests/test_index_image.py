"""Serialized DiskANN index images: the host-side parser against the oracle's restatement of
the reference's reader (rust_lib/src/file_format.rs:3-18, rust_lib/src/index_manager.rs:513-533,
560-668), and, on a GPU, the loader that registers the segments as device tables."""
import numpy as np
import pytest


def _image(oracle, n=300, d=48, deg=8, ne=2, metric=0, with_sq8=True, seed=1):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n, d)).astype(np.float32)
    adj = rng.integers(0, n, (n, deg)).astype(np.uint32)
    adj[rng.random((n, deg)) < 0.3] = 0xFFFFFFFF
    entry = rng.integers(0, n, ne).astype(np.uint32)
    sq8 = None
    if with_sq8:
        mins, scale = oracle.sq8_train(x)
        sq8 = (mins, scale, oracle.sq8_encode(x, mins, scale))
    return oracle.write_diskann_image(x, adj, entry, metric, 77, sq8), x, adj, entry, sq8


@pytest.mark.parametrize("with_sq8", [True, False])
@pytest.mark.parametrize("metric", [0, 1])
def test_parser_agrees_with_the_oracle(pkg, oracle, with_sq8, metric):
    image, x, adj, entry, sq8 = _image(oracle, metric=metric, with_sq8=with_sq8)
    want = oracle.parse_diskann_image(image)
    info = pkg.diskann_bridge.parse_index(image)
    assert (info.num_vectors, info.dimension, info.max_degree, info.num_entry_points) == (300, 48, 8, 2)
    assert info.metric == metric and info.build_complexity == 77
    assert info.entry_points_offset == 32 and info.vectors_offset == 32 + 8
    assert info.adjacency_offset == info.vectors_offset + x.nbytes
    assert info.standard_size == want["standard_size"]
    assert np.frombuffer(image, "<f4", x.size, info.vectors_offset).tobytes() == want["vectors"].tobytes()
    assert np.frombuffer(image, "<u4", adj.size, info.adjacency_offset).tobytes() == adj.tobytes()
    assert bool(info.has_sq8) == with_sq8
    if with_sq8:
        mins, scale, codes = want["sq8"]
        assert np.frombuffer(image, "<f4", 48, info.sq8_min_offset).tobytes() == mins.tobytes()
        assert np.frombuffer(image, "<f4", 48, info.sq8_scale_offset).tobytes() == scale.tobytes()
        assert info.sq8_codes_size == codes.size
        assert image[info.sq8_codes_offset:info.sq8_codes_offset + codes.size] == codes.tobytes()


def test_parser_rejects_bad_images(pkg, oracle):
    image, *_ = _image(oracle)
    br = pkg.diskann_bridge
    for bad in (image[:20], b"NNAD" + image[4:], image[:4] + (3).to_bytes(4, "little") + image[8:],
                image[:len(image) // 3]):
        with pytest.raises(pkg.AnnCudaError):
            br.parse_index(bad)
    std = br.parse_index(image).standard_size
    with pytest.raises(pkg.AnnCudaError):      # trailer cut inside the codes
        br.parse_index(image[:-10])
    wrong_dim = bytearray(image)
    wrong_dim[std + 4:std + 8] = (47).to_bytes(4, "little")
    with pytest.raises(pkg.AnnCudaError):
        br.parse_index(bytes(wrong_dim))
    # bytes after the adjacency that are not a trailer are ignored, as by the reference
    assert not br.parse_index(image[:std] + b"junk-junk").has_sq8


@pytest.mark.gpu
def test_loaded_tables_score_like_the_oracle(pkg, oracle, tmp_path):
    image, x, adj, entry, sq8 = _image(oracle, n=5000, d=64, seed=3)
    path = tmp_path / "index.diskann"
    path.write_bytes(image)
    rng = np.random.default_rng(9)
    q = rng.standard_normal((4, 64)).astype(np.float32)
    ids = rng.integers(0, 5000, 4 * 50).astype(np.uint32)
    qm = np.repeat(np.arange(4, dtype=np.uint32), 50)
    for source in (image, path):
        info, vec, codes = pkg.diskann_bridge.load_index(source)
        assert info.num_vectors == 5000 and codes is not None
        got = vec.batch_distances_by_id(q, ids, qm, 0)
        want = oracle.batch_distances_by_id(x, q, ids, qm, 0, exact=True)
        np.testing.assert_allclose(got, want, rtol=1e-5)
        got8 = codes.batch_distances_by_id(q, ids, qm, 0)
        want8 = oracle.sq8_batch_distances_by_id(sq8[2], sq8[0], sq8[1], q, ids, qm, 0, exact=True)
        np.testing.assert_allclose(got8, want8, rtol=1e-4)
        vec.close()
        codes.close()
