"""The K/V page allocator on the host (no GPU): LIFO order with page 0 first, exhaustion, shared pages returning to the
stack with their last holder only -- the observable behaviour of the reference's GlobalKvPagePool
(src/qwen_native_backend.cpp:1155-1265: free stack, pinned pages of cached prefixes never handed out)."""
import threading


def test_lifo_order_and_exhaustion(qb):
    L = qb.lib()
    pool = L.qb_page_pool_create(5)
    assert L.qb_page_pool_free_count(pool) == 5
    got = [L.qb_page_pool_alloc(pool) for _ in range(5)]
    assert got == [0, 1, 2, 3, 4]                       # page 0 first
    assert L.qb_page_pool_alloc(pool) == -1             # exhausted: reported, nothing changes
    assert L.qb_page_pool_free_count(pool) == 0
    assert L.qb_page_pool_drop(pool, 3) == 0 and L.qb_page_pool_drop(pool, 1) == 0
    assert L.qb_page_pool_alloc(pool) == 1              # most recently freed first
    assert L.qb_page_pool_alloc(pool) == 3
    assert L.qb_page_pool_drop(pool, 9) == -1 and L.qb_page_pool_drop(pool, -1) == -1
    L.qb_page_pool_destroy(pool)


def test_shared_pages_outlive_their_first_holder(qb):
    L = qb.lib()
    pool = L.qb_page_pool_create(4)
    a = [L.qb_page_pool_alloc(pool) for _ in range(3)]          # a request's pages
    assert all(L.qb_page_pool_share(pool, p) == 1 for p in a[:2])   # a prefix entry holds the first two as well
    for p in reversed(a):                                       # the request retires
        L.qb_page_pool_drop(pool, p)
    assert L.qb_page_pool_free_count(pool) == 2                 # page 2 and the never-used page 3
    assert L.qb_page_pool_alloc(pool) == 2                      # the shared pages are not handed out
    assert L.qb_page_pool_alloc(pool) == 3
    assert L.qb_page_pool_alloc(pool) == -1
    assert L.qb_page_pool_share(pool, 0) == 1                   # a second request attaches the prefix
    assert L.qb_page_pool_drop(pool, 0) == 1 and L.qb_page_pool_drop(pool, 0) == 0   # ... retires; the entry is evicted
    assert L.qb_page_pool_alloc(pool) == 0
    assert L.qb_page_pool_share(pool, 1) == 1 and L.qb_page_pool_drop(pool, 1) == 1
    L.qb_page_pool_drop(pool, 1)
    assert L.qb_page_pool_share(pool, 1) == 0                   # a free page cannot be shared
    L.qb_page_pool_destroy(pool)


def test_pool_is_thread_safe(qb):
    L = qb.lib()
    n = 4096
    pool = L.qb_page_pool_create(n)
    got = [[] for _ in range(8)]

    def work(i):
        for _ in range(n // 8):
            got[i].append(L.qb_page_pool_alloc(pool))

    th = [threading.Thread(target=work, args=(i,)) for i in range(8)]
    [t.start() for t in th]
    [t.join() for t in th]
    flat = sorted(p for g in got for p in g)
    assert flat == list(range(n))                               # every page exactly once
    assert L.qb_page_pool_alloc(pool) == -1
    L.qb_page_pool_destroy(pool)
