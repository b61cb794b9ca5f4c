from .pages import PAGE_TOKENS, CacheError, GroupPlan, PagePool, SequencePages, SlotTable
