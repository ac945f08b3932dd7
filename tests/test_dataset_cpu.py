"""Legion-format dataset files and the meta_config line, without a GPU (pin=False)."""
import os

import numpy as np
import pytest

import legion_ibp_b200 as L
from conftest import small_graph


def write_dataset(d, n=500, f=7, with_partition=False, seed=0):
    rng = np.random.default_rng(seed)
    indptr, indices = small_graph(n, 4000, seed)
    feats = rng.standard_normal((n, f)).astype(np.float32)
    labels = rng.integers(0, 10, n).astype(np.int32)
    perm = rng.permutation(n).astype(np.int32)
    train, valid, test = perm[:200], perm[200:260], perm[260:400]
    os.makedirs(d, exist_ok=True)
    indptr.astype(np.int64).tofile(os.path.join(d, "edge_src"))
    indices.astype(np.int32).tofile(os.path.join(d, "edge_dst"))
    feats.tofile(os.path.join(d, "features"))
    labels.tofile(os.path.join(d, "labels"))
    train.tofile(os.path.join(d, "trainingset"))
    valid.tofile(os.path.join(d, "validationset"))
    test.tofile(os.path.join(d, "testingset"))
    part = rng.integers(0, 4, n).astype(np.int32)
    if with_partition:
        part.tofile(os.path.join(d, "partition"))
    return dict(indptr=indptr, indices=indices, feats=feats, labels=labels, train=train, valid=valid, test=test, part=part)


def meta_for(d, ref, f=7):
    m = L.MetaConfig()
    m.dataset_path = (str(d) + "/").encode()
    m.feature_path = (str(d) + "/").encode()
    m.raw_batch_size = 32
    m.node_num = len(ref["indptr"]) - 1
    m.edge_num = len(ref["indices"])
    m.float_feature_len = f
    m.training_set_num, m.validation_set_num, m.testing_set_num = len(ref["train"]), len(ref["valid"]), len(ref["test"])
    m.cache_memory = 123456789
    m.epoch = 3
    return m


def test_meta_config_round_trip_and_reference_line(tmp_path):
    ref = write_dataset(tmp_path / "ds")
    m = meta_for(tmp_path / "ds", ref)
    path = str(tmp_path / "meta_config")
    m.write(path)
    line = open(path).read().split()
    # "path batch nodes edges feature_dim ntrain nvalid ntest cache_bytes epochs feature_path"
    assert line[1:10] == ["32", str(m.node_num), str(m.edge_num), "7", "200", "60", "140", "123456789", "3"]
    back = L.MetaConfig.read(path)
    for name, _ in L.MetaConfig._fields_:
        assert getattr(back, name) == getattr(m, name), name
    # the 10-field form written by older launchers: the feature path defaults to the dataset path
    open(path, "w").write(" ".join(line[:10]) + "\n")
    assert L.MetaConfig.read(path).feature_path == m.dataset_path
    open(path, "w").write("only three fields\n")
    with pytest.raises(L.LegionError):
        L.MetaConfig.read(path)
    with pytest.raises(L.LegionError):
        L.MetaConfig.read(str(tmp_path / "missing"))


@pytest.mark.parametrize("with_partition", [False, True])
def test_load_and_split(tmp_path, with_partition):
    ref = write_dataset(tmp_path / "ds", with_partition=with_partition)
    ds = L.Dataset(meta_for(tmp_path / "ds", ref), pin=False)
    np.testing.assert_array_equal(ds.indptr, ref["indptr"])
    np.testing.assert_array_equal(ds.indices, ref["indices"])
    np.testing.assert_array_equal(ds.features, ref["feats"])
    np.testing.assert_array_equal(ds.labels, ref["labels"])
    for world in (1, 2, 4):
        seen = []
        for rank in range(world):
            for mode, key in ((L.TRAINMODE, "train"), (L.VALIDMODE, "valid"), (L.TESTMODE, "test")):
                ids, lab = ds.split(mode, world, rank)
                src = ref[key]
                if mode == L.TRAINMODE and with_partition:
                    want = src[ref["part"][src] == rank]   # owners >= world are dropped, as in the reference
                else:
                    want = src[src % world == rank]
                np.testing.assert_array_equal(ids, want)
                np.testing.assert_array_equal(lab, ref["labels"][want])
                if mode == L.TRAINMODE:
                    seen += list(ids)
        if not with_partition:
            assert sorted(seen) == sorted(ref["train"].tolist())
    ds.close()


def test_load_rejects_inconsistent_files(tmp_path):
    ref = write_dataset(tmp_path / "ds")
    m = meta_for(tmp_path / "ds", ref)
    m.edge_num += 1
    with pytest.raises(L.LegionError, match="edge_dst"):
        L.Dataset(m, pin=False)
    m = meta_for(tmp_path / "ds", ref)
    os.remove(tmp_path / "ds" / "labels")
    with pytest.raises(L.LegionError, match="cannot open file"):
        L.Dataset(m, pin=False)
    ref = write_dataset(tmp_path / "ds2")
    np.array([9999], np.int32).tofile(tmp_path / "ds2" / "testingset")
    m = meta_for(tmp_path / "ds2", ref)
    m.testing_set_num = 1
    with pytest.raises(L.LegionError, match="outside"):
        L.Dataset(m, pin=False)
