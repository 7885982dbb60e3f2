import json
import os

import pytest

from recsdk_b200.common import (DirectoryValidator, ValidationError, Validator, bind_cpu, cores_for_rank, int_safe_check, logger,
                                path_safe_check, rank_info_from_env, rank_info_from_table, str_safe_check)


def test_validators():
    assert int_safe_check("n", 3, 1, 8) == 3
    with pytest.raises(ValidationError):
        int_safe_check("n", 9, 1, 8)
    with pytest.raises(ValidationError):
        int_safe_check("n", True, 0, 8)
    assert str_safe_check("name", "table_0", r"^[A-Za-z0-9_]+$") == "table_0"
    with pytest.raises(ValidationError):
        path_safe_check("p", "/tmp/../etc")
    assert Validator([1, 2], "xs").check_type(list).check_length(1, 4).is_valid()
    assert not DirectoryValidator("/definitely/not/here").check_exists().is_valid()


def test_rank_info(tmp_path):
    ri = rank_info_from_env({"WORLD_SIZE": "16", "RANK": "11", "LOCAL_WORLD_SIZE": "8", "MASTER_ADDR": "10.0.0.1"})
    assert (ri.local_rank, ri.node_rank, ri.device_id, ri.host) == (3, 1, 3, "10.0.0.1")
    with pytest.raises(ValueError):
        rank_info_from_env({"WORLD_SIZE": "2", "RANK": "2"})
    table = {"server_list": [{"server_id": "a", "device": [{"device_id": "0", "rank_id": "0"}, {"device_id": "1", "rank_id": "1"}]},
                             {"server_id": "b", "device": [{"device_id": "0", "rank_id": "2"}, {"device_id": "1", "rank_id": "3"}]}]}
    p = tmp_path / "ranktable.json"
    p.write_text(json.dumps(table))
    ri = rank_info_from_table(str(p), 3)
    assert (ri.world_size, ri.local_rank, ri.device_id, ri.host) == (4, 1, 1, "b")


def test_bind_cpu_restores_affinity():
    before = os.sched_getaffinity(0)
    assert cores_for_rank(1, 2, [0, 1, 2, 3]) == [2, 3] and cores_for_rank(0, 2, [0, 1, 2, 3], reserve=1) == [1]

    @bind_cpu(local_rank=0, local_world_size=1)
    def inside():
        return os.sched_getaffinity(0)

    assert inside() <= before and os.sched_getaffinity(0) == before
    logger.set_level("ERROR")
    logger.info("not shown")


def test_typed_validators_and_decorator(tmp_path):
    import os

    import pytest

    from recsdk_b200.common.validator import (AndValidator, ClassValidator, Convert2intValidator, FileValidator, FloatValidator,
                                              IntValidator, ListValidator, OptionalIntValidator, OptionValidator, OrValidator,
                                              StringValidator, ValidationError, para_checker_decorator)

    assert IntValidator(5, "n", 1, 8).validate() == 5
    for bad in (True, 9, 5.0, "5"):
        assert not IntValidator(bad, "n", 1, 8).is_valid()
    assert FloatValidator(0.5, "lr", 0.0, 1.0, "(]").is_valid() and not FloatValidator(0.0, "lr", 0.0, 1.0, "(]").is_valid()
    assert OptionalIntValidator(None, "k", 0, 3).validate() is None and not OptionalIntValidator(7, "k", 0, 3).is_valid()
    assert Convert2intValidator("12", "port", 1, 65535).validate() == 12 and not Convert2intValidator("x", "port").is_valid()
    assert ListValidator([1, 2, 3], "dims", IntValidator, 1, 4, min_value=1).is_valid()
    assert not ListValidator([1, 0], "dims", IntValidator, min_value=1).is_valid()
    assert OptionValidator("mean", "pooling", ["sum", "mean"]).is_valid() and not OptionValidator("max", "pooling", ["sum", "mean"]).is_valid()
    assert ClassValidator(3, "x", (int, float)).is_valid() and not ClassValidator("3", "x", int).is_valid()
    either = OrValidator("auto", "threads", [IntValidator("auto", "threads", 1), OptionValidator("auto", "threads", ["auto"])])
    assert either.is_valid()
    assert not AndValidator("a" * 9, "name", [StringValidator("a" * 9, "name", 8)]).is_valid()
    f = tmp_path / "w.bin"
    f.write_bytes(b"x" * 10)
    os.chmod(f, 0o640)
    ok = FileValidator(str(f), "ckpt").check_not_soft_link().check_file_size(100).check_user_group().check_file_mode()
    assert ok.is_valid()
    os.chmod(f, 0o666)
    assert not FileValidator(str(f), "ckpt").check_file_mode().is_valid()
    link = tmp_path / "l.bin"
    os.symlink(f, link)
    assert not FileValidator(str(link), "ckpt").check_not_soft_link().is_valid()

    @para_checker_decorator([("lr", FloatValidator, {"min_value": 0.0, "max_value": 1.0}),
                             (["rows", "dim"], IntValidator, {"min_value": 1})])
    def make(rows, dim=8, lr=0.1):
        return rows * dim

    assert make(4) == 32 and make(4, dim=2, lr=0.5) == 8
    with pytest.raises(ValidationError):
        make(0)
    with pytest.raises(ValidationError):
        make(4, lr=2.0)
