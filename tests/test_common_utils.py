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


def test_reference_named_getters_and_checks(tmp_path, monkeypatch, capsys):
    """Names of ``rec_sdk_common``: rank / device getters (``communication/hccl/hccl_info.py``), class / dir / file safe checks
    (``validator/safe_checker.py``), the class-level logger (``log/log.py``), CPU binding helpers (``perf_factory/bind_cpu.py``)."""
    import json
    import os

    import pytest

    from recsdk_b200.common import (ValidationError, bind_cpu_task, class_safe_check, dir_safe_check, file_safe_check,
                                    get_available_cpu_num_and_range, get_device_id, get_device_list, get_local_rank_size, get_min_device_id,
                                    get_rank_id, get_rank_size, get_rank_to_device_dict)
    from recsdk_b200.common.log import LoggingProxy

    for k in ("RANK", "WORLD_SIZE", "LOCAL_WORLD_SIZE", "OMPI_COMM_WORLD_RANK", "OMPI_COMM_WORLD_SIZE", "OMPI_COMM_WORLD_LOCAL_SIZE",
              "RANK_TABLE_FILE", "CUDA_VISIBLE_DEVICES", "LOCAL_RANK"):
        monkeypatch.delenv(k, raising=False)
    with pytest.raises(RuntimeError):
        get_rank_id()
    monkeypatch.setenv("OMPI_COMM_WORLD_RANK", "5")                      # Open MPI's names serve when torchrun's are absent
    monkeypatch.setenv("OMPI_COMM_WORLD_SIZE", "8")
    monkeypatch.setenv("OMPI_COMM_WORLD_LOCAL_SIZE", "4")
    assert (get_rank_id(), get_rank_size(), get_local_rank_size()) == (5, 8, 4)
    monkeypatch.setenv("RANK", "6")
    assert get_rank_id() == 6
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "4,5,6,7")
    assert get_rank_to_device_dict() == {0: 4, 1: 5, 2: 6, 3: 7} and get_device_id() == 6 and get_min_device_id() == 4
    assert get_device_list() == [4, 5, 6, 7]
    monkeypatch.setenv("WORLD_SIZE", "zero")
    with pytest.raises(ValueError):
        get_rank_size()
    monkeypatch.setenv("WORLD_SIZE", "0")
    with pytest.raises(ValueError):
        get_rank_size()
    table = {"server_list": [{"server_id": "h", "device": [{"device_id": "3", "rank_id": "0"}, {"device_id": "1", "rank_id": "6"}]}]}
    p = tmp_path / "ranks.json"
    p.write_text(json.dumps(table))
    monkeypatch.setenv("RANK_TABLE_FILE", str(p))
    assert get_rank_to_device_dict() == {0: 3, 6: 1} and get_device_id() == 1 and get_min_device_id() == 1

    assert class_safe_check("topology", 3, (int, float)) == 3 and class_safe_check("x", "s", str) == "s"
    with pytest.raises(ValidationError, match="instance of int/float"):
        class_safe_check("topology", "3", (int, float))
    d = tmp_path / "data"
    d.mkdir()
    assert dir_safe_check("dir", str(d)) == str(d)
    os.symlink(str(d), str(tmp_path / "ln"))
    for bad in (str(tmp_path / "ln"), str(tmp_path / "missing"), "", None):
        with pytest.raises(ValidationError):
            dir_safe_check("dir", bad)
    f = d / "weights.bin"
    f.write_bytes(b"12345678")
    os.chmod(str(f), 0o600)
    assert file_safe_check("file", str(f)) == str(f)
    os.chmod(str(f), 0o666)
    with pytest.raises(ValidationError, match="permission bits"):
        file_safe_check("file", str(f))
    os.chmod(str(f), 0o600)
    with pytest.raises(ValidationError, match="size"):
        file_safe_check("file", str(f), max_size=4)
    with pytest.raises(ValidationError):
        file_safe_check("file", str(d))

    import logging

    class Keep(logging.Handler):
        def __init__(self):
            super().__init__()
            self.records = []

        def emit(self, record):
            self.records.append(record)

    LoggingProxy.set_instance("WARNING")
    keep = Keep()
    LoggingProxy._instance.addHandler(keep)
    try:
        LoggingProxy.info("quiet")
        LoggingProxy.warning("loud %s", "enough")
        try:
            raise KeyError("k")
        except KeyError:
            LoggingProxy.exception("with a traceback")
    finally:
        LoggingProxy._instance.removeHandler(keep)
    assert [r.getMessage() for r in keep.records] == ["loud enough", "with a traceback"]
    assert keep.records[1].exc_info is not None and keep.records[1].levelname == "ERROR"
    with pytest.raises(ValueError):
        LoggingProxy.set_instance("chatty")
    LoggingProxy.set_instance("INFO")

    n, ranges = get_available_cpu_num_and_range()
    assert n == len(os.sched_getaffinity(0)) and all(lo <= hi for lo, hi in ranges) and len(ranges) >= 1
    monkeypatch.setenv("LOCAL_WORLD_SIZE", "1")
    assert bind_cpu_task() is None
    before = os.sched_getaffinity(0)
    if len(before) >= 2:
        monkeypatch.setenv("LOCAL_WORLD_SIZE", "2")
        monkeypatch.setenv("LOCAL_RANK", "1")
        try:
            got = bind_cpu_task()
            assert got and set(got) < set(before)
        finally:
            os.sched_setaffinity(0, before)
