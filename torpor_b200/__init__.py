"""B200-native model swap engine behind Torpor's MemoryManager interface."""
