"""Byte counters printed every `verbose_freq` minibatches (runtime/runtime_utilities.py:4-28)."""


class RuntimeStats:
    def __init__(self, forward):
        self.forward = forward
        self.stats = {}
        self.reset_stats()

    def reset_stats(self):
        self.stats = {
            'compute_time': 0.0,
            'send_tensors': 0.0,
            'send_tensors_size': 0,
            'receive_tensors': 0.0,
            'receive_tensors_size': 0,
        }

    def print_stats(self):
        direction = "Forward" if self.forward else "Backward"
        print("%s Stats:" % direction)
        for key in sorted(self.stats):
            units = "bytes" if key.endswith("_size") else "seconds"
            print("\t%s %.3f %s" % (key, self.stats[key], units))
