"""Session sharding across GPUs: the step partitions by session with weights replicated, so a
box of N GPUs is N engines that never exchange data during a step. Rows of different slots share
nothing but the read-only weights (Sources/SploshRuntime/Engine.swift:7-10, 1383-1385); the only
traffic is the host gathering token ids afterwards."""


def assign_sessions(session_ids, world_size):
    """Round-robin assignment: shard r takes sessions r, r + N, r + 2N, ... Returns a list of lists."""
    shards = [[] for _ in range(world_size)]
    for index, sid in enumerate(session_ids):
        shards[index % world_size].append(sid)
    return shards


def local_slot(session_index, world_size):
    """The slot a session takes on its shard's engine."""
    return session_index // world_size


def gather_ids(local_ids, dist=None):
    """All shards' (session id, token ids) pairs on every rank, ordered by session id. `dist` is
    torch.distributed (any backend) or None for a single process."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return sorted(local_ids)
    gathered = [None] * dist.get_world_size()
    dist.all_gather_object(gathered, local_ids)
    return sorted(pair for part in gathered for pair in part)
