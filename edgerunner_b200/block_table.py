"""Host-side page allocator for the paged KV layout.

The reference has no paging (one contiguous ring per layer, Sources/EdgeRunnerMetal/KVCache.swift:357-370);
this is the block-table allocator the CUDA backend's host layer owns: a free list over a shared page pool,
one block table (list of page ids) per sequence, grown a page at a time as the sequence gets longer.
"""


class OutOfPages(RuntimeError):
    pass


class BlockTableAllocator:
    def __init__(self, num_pages, page_size, free_order=None):
        if page_size <= 0 or page_size % 16:
            raise ValueError("page_size must be a positive multiple of 16")
        self.num_pages, self.page_size = int(num_pages), int(page_size)
        order = list(range(self.num_pages)) if free_order is None else [int(p) for p in free_order]
        if sorted(order) != list(range(self.num_pages)):
            raise ValueError("free_order must be a permutation of the page pool")
        self._free = order[::-1]          # pop() hands pages out in free_order
        self._tables = {}

    @property
    def free_pages(self):
        return len(self._free)

    def pages_for(self, tokens):
        return (int(tokens) + self.page_size - 1) // self.page_size

    def block_table(self, seq):
        return list(self._tables.get(seq, ()))

    def ensure(self, seq, tokens):
        """Grow the table of `seq` so that it covers `tokens` tokens; returns the table."""
        table = self._tables.setdefault(seq, [])
        need = self.pages_for(tokens) - len(table)
        if need > len(self._free):
            raise OutOfPages("sequence %r needs %d more pages, %d free" % (seq, need, len(self._free)))
        for _ in range(max(need, 0)):
            table.append(self._free.pop())
        return list(table)

    def release(self, seq):
        for p in reversed(self._tables.pop(seq, [])):
            self._free.append(p)
