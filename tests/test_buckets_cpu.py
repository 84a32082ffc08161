"""Padded-size arithmetic of the neighbour list against the reference's known answers
(``tests/cpu/test_neighbors.py:178-198`` of the reference; the functions restate ``fastmace/neighbors/buckets.py:19-34``)."""
import pytest

from fastmace_b200.neighbours import edge_bucket, edge_capacity, round_up_edges


@pytest.mark.parametrize("count,fraction,multiple,expected", [
    (6912, 0.0, 256, 256), (6912, 0.05, 256, 512), (51084, 0.05, 256, 2560), (100, 0.05, 256, 256), (6912, 0.05, 128, 384)])
def test_edge_bucket(count, fraction, multiple, expected):
    assert edge_bucket(count, fraction, multiple) == expected


@pytest.mark.parametrize("count,capacity,bucket,expected", [
    (7000, 10**6, 512, 7168), (7168, 10**6, 512, 7168), (0, 10**6, 512, 512), (7000, 7100, 512, 7100), (7000, 10**6, 256, 7168)])
def test_round_up_edges(count, capacity, bucket, expected):
    assert round_up_edges(count, capacity, bucket) == expected


@pytest.mark.parametrize("needed,headroom,multiple,expected", [
    (1000, 1.15, 256, 1280), (1024, 1.0, 256, 1024), (1, 1.15, 256, 256), (1000, 1.15, 100, 1200)])
def test_edge_capacity(needed, headroom, multiple, expected):
    assert edge_capacity(needed, headroom, multiple) == expected
