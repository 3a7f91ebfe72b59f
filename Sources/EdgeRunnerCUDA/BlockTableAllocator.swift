// Host-side page allocator of the paged KV layout: a free list over the shared page pool and one block table (list of page
// ids) per sequence, grown a page at a time.  The reference has no paging (one contiguous ring per layer,
// Sources/EdgeRunnerMetal/KVCache.swift:357-370); policy lives here, above the C ABI, which only stores the tables
// (er_kv_set_block_table).  Same behaviour as edgerunner_b200/block_table.py and edgerunner::BlockTableAllocator.
// Uncompiled in this repository.
public struct OutOfPages: Error, Sendable { public let sequence: Int, needed: Int, free: Int }

public struct BlockTableAllocator: Sendable {
    public let numPages: Int
    public let pageSize: Int
    private var free: [Int32]                 // popLast() hands pages out in `freeOrder`
    private var tables: [Int: [Int32]] = [:]

    public init(numPages: Int, pageSize: Int, freeOrder: [Int32]? = nil) {
        precondition(pageSize > 0 && pageSize % 16 == 0, "pageSize must be a positive multiple of 16")
        let order = freeOrder ?? (0..<Int32(numPages)).map { $0 }
        precondition(order.sorted() == (0..<Int32(numPages)).map { $0 }, "freeOrder must be a permutation of the page pool")
        self.numPages = numPages
        self.pageSize = pageSize
        self.free = order.reversed()
    }
    public var freePages: Int { free.count }
    public func pages(for tokens: Int) -> Int { (tokens + pageSize - 1) / pageSize }
    public func blockTable(_ sequence: Int) -> [Int32] { tables[sequence] ?? [] }

    /// Grows the table of `sequence` so that it covers `tokens` tokens and returns it.
    public mutating func ensure(_ sequence: Int, tokens: Int) throws -> [Int32] {
        var table = tables[sequence] ?? []
        let need = pages(for: tokens) - table.count
        guard need <= free.count else { throw OutOfPages(sequence: sequence, needed: need, free: free.count) }
        for _ in 0..<max(need, 0) { table.append(free.removeLast()) }
        tables[sequence] = table
        return table
    }
    public mutating func release(_ sequence: Int) {
        for p in (tables.removeValue(forKey: sequence) ?? []).reversed() { free.append(p) }
    }
}
