"""Throughput and memory bookkeeping of a training / evaluation run: the interface of the reference's
``PerformanceCounter`` (pydtnn/utils/performance_counter.py:25-153: the model records one (seconds, samples) pair per
batch, keyed by epoch or evaluation round, and reports totals, throughput, a throughput extrapolated from the last
half of each epoch, and the host's resident-set size).  Times here are host wall-clock seconds around a whole step
including its read-back, as in the reference (pydtnn/model.py:576-590)."""
import resource
from collections import defaultdict


class PerformanceCounter:
    TRAINING, TESTING = range(2)

    def __init__(self):
        self._records = {self.TRAINING: defaultdict(list), self.TESTING: defaultdict(list)}

    # -- recording ---------------------------------------------------------------------------------
    def add_training_time_and_batch_size(self, epoch, elapsed_time, batch_size):
        self._add(self.TRAINING, epoch, elapsed_time, batch_size)

    def add_testing_time_and_batch_size(self, test_round, elapsed_time, batch_size):
        self._add(self.TESTING, test_round, elapsed_time, batch_size)

    def _add(self, where, key, elapsed_time, batch_size):
        usage = resource.getrusage(resource.RUSAGE_SELF).ru_maxrss + resource.getrusage(resource.RUSAGE_CHILDREN).ru_maxrss
        self._records[where][key].append((float(elapsed_time), int(batch_size), usage))        # KiB on Linux

    # -- totals ------------------------------------------------------------------------------------
    def _total(self, where, field, last_half=False):
        """Sum of a field over all rounds; with ``last_half`` each round is extrapolated from its second half (the
        first steps of an epoch carry warm-up costs)."""
        total = 0.0
        for rows in self._records[where].values():
            vals = [r[field] for r in rows]
            if last_half:
                tail = vals[len(vals) // 2:]
                if tail:
                    total += sum(tail) * len(vals) / len(tail)
            else:
                total += sum(vals)
        return total

    def _throughput(self, where, last_half=False):
        t = self._total(where, 0, last_half)
        return self._total(where, 1, last_half) / t if t > 0 else 0.0

    def _memory(self, where):
        return [r[2] for rows in self._records[where].values() for r in rows]

    num_epochs = property(lambda self: len(self._records[self.TRAINING]))
    num_evaluations = property(lambda self: len(self._records[self.TESTING]))
    training_time = property(lambda self: self._total(self.TRAINING, 0))
    training_time_estimated_from_last_half_of_each_epoch = property(lambda self: self._total(self.TRAINING, 0, True))
    training_throughput = property(lambda self: self._throughput(self.TRAINING))
    training_throughput_only_last_half_of_each_epoch = property(lambda self: self._throughput(self.TRAINING, True))
    training_maximum_memory = property(lambda self: max(self._memory(self.TRAINING), default=0))
    training_mean_memory = property(lambda self: (lambda m: sum(m) / len(m) if m else 0.0)(self._memory(self.TRAINING)))
    testing_time = property(lambda self: self._total(self.TESTING, 0))
    testing_throughput = property(lambda self: self._throughput(self.TESTING))
    testing_maximum_memory = property(lambda self: max(self._memory(self.TESTING), default=0))
    testing_mean_memory = property(lambda self: (lambda m: sum(m) / len(m) if m else 0.0)(self._memory(self.TESTING)))

    def report(self):
        """The lines ``print_report`` prints, as a list of strings."""
        out = []
        if self.num_epochs:
            out += ["Performance counter training report",
                    f"Training time (from model): {self.training_time:5.4f} s",
                    f"Training time per epoch (from model): {self.training_time / self.num_epochs:5.4f} s",
                    f"Training throughput (from model): {self.training_throughput:5.4f} samples/s",
                    f"Training time (from model, estimated from last half of each epoch): "
                    f"{self.training_time_estimated_from_last_half_of_each_epoch:5.4f} s",
                    f"Training throughput (from model, from last half of each epoch): "
                    f"{self.training_throughput_only_last_half_of_each_epoch:5.4f} samples/s",
                    f"Training maximum memory allocated: {self.training_maximum_memory / 1024:.2f} MiB",
                    f"Training mean memory allocated: {self.training_mean_memory / 1024:.2f} MiB"]
        if self.num_evaluations:
            out += ["Performance counter testing report",
                    f"Testing time (from model): {self.testing_time:5.4f} s",
                    f"Testing throughput (from model): {self.testing_throughput:5.4f} samples/s",
                    f"Testing maximum memory allocated: {self.testing_maximum_memory / 1024:.2f} MiB",
                    f"Testing mean memory allocated: {self.testing_mean_memory / 1024:.2f} MiB"]
        return out

    def print_report(self):
        print("\n".join(self.report()))
