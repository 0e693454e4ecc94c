"""The diagnostic trace names kernels from the sources: every dependency wait must map to the __global__ function around it."""
import re

from inferulm_b200 import trace


def test_every_dependency_wait_maps_to_a_kernel():
    sites = trace.call_sites()
    assert len(sites) >= 30
    for (fid, line), name in sites.items():
        assert re.fullmatch(r"\w+_kernel", name), (fid, line, name)
    names = set(sites.values())
    for k in ("wgemm_kernel", "tgemm_kernel", "gdn_layer_kernel", "gdn_commit_kernel", "attn_verify_kernel", "topk_filter_kernel",
              "accept_kernel", "commit_kernel", "rms_norm_zc_kernel"):
        assert k in names


def test_file_id_is_fnv1a_of_the_base_name():
    assert trace.file_id("") == 2166136261
    assert trace.file_id("a") == ((2166136261 ^ ord("a")) * 16777619) & 0xFFFFFFFF
    assert len({trace.file_id(u + ".cu") for u in trace.UNITS}) == len(trace.UNITS)
