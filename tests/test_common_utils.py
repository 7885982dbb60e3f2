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
