"""List-based statement of the per-slot KV-cache semantics (no numeric library).

Mirrors the reference's llm/cache_reference.py:4-67: `exact_int`, `KVCache` with a
transactional `append_batch`, `reset`, `read`, and `causal_keys`.  Storage is
[slot][layer] -> list of per-position entries; what is stored per position is opaque.  It
states what the paged device cache must do: append at each slot's own length, isolate slots,
reject a whole batch when any member is invalid, never alias caller data.
"""
import copy


def exact_int(value, name, low, high):
    if type(value) is not int or not low <= value <= high:
        raise ValueError(f"{name} must be an integer in [{low},{high}]")
    return value


class KVCache:
    def __init__(self, slots, layers, capacity):
        self.slots = exact_int(slots, "slots", 1, 1024)
        self.layers = exact_int(layers, "layers", 1, 1024)
        self.capacity = exact_int(capacity, "capacity", 1, 1024)
        self.lengths = [0] * slots
        self.k = [[[] for _ in range(layers)] for _ in range(slots)]
        self.v = [[[] for _ in range(layers)] for _ in range(slots)]

    def _slot(self, slot):
        return exact_int(slot, "slot", 0, self.slots - 1)

    def reset(self, slot):
        slot = self._slot(slot)
        self.lengths[slot] = 0
        self.k[slot] = [[] for _ in range(self.layers)]
        self.v[slot] = [[] for _ in range(self.layers)]

    def append_batch(self, slots, keys, values):
        """keys/values: per request, per layer, a sequence of new positions.  All or nothing."""
        if not slots or len(slots) != len(keys) or len(slots) != len(values):
            raise ValueError("nonempty matched batch required")
        targets = [self._slot(s) for s in slots]
        if len(set(targets)) != len(targets):
            raise ValueError("duplicate slot")
        counts = []
        for slot, k, v in zip(targets, keys, values):
            if len(k) != self.layers or len(v) != self.layers:
                raise ValueError("one key/value sequence per layer required")
            n = len(k[0])
            if n <= 0 or any(len(seq) != n for seq in list(k) + list(v)):
                raise ValueError("matched positive append lengths required")
            if self.lengths[slot] + n > self.capacity:
                raise ValueError("cache capacity exceeded")
            counts.append(n)
        own_k, own_v = copy.deepcopy((keys, values))          # nothing mutated before this point
        for slot, k, v, n in zip(targets, own_k, own_v, counts):
            for layer in range(self.layers):
                self.k[slot][layer].extend(k[layer])
                self.v[slot][layer].extend(v[layer])
            self.lengths[slot] += n

    def read(self, slot, layer):
        slot = self._slot(slot)
        layer = exact_int(layer, "layer", 0, self.layers - 1)
        return copy.deepcopy((self.k[slot][layer], self.v[slot][layer]))


def causal_keys(query_index, query_offset, valid_length):
    """Keys visible to query `query_index` of an append that starts at `query_offset`."""
    exact_int(query_index, "query_index", 0, 1023)
    exact_int(query_offset, "query_offset", 0, 1023)
    exact_int(valid_length, "valid_length", 0, 1024)
    return range(min(valid_length, query_offset + query_index + 1))
