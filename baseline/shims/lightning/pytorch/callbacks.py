class Callback:
    """Hook container with the no-op hooks of Lightning's ``Callback`` that the reference's trainers invoke."""

    def setup(self, *args, **kwargs):
        pass

    def teardown(self, *args, **kwargs):
        pass

    def on_fit_start(self, *args, **kwargs):
        pass

    def on_fit_end(self, *args, **kwargs):
        pass

    def on_train_start(self, *args, **kwargs):
        pass

    def on_train_end(self, *args, **kwargs):
        pass

    def on_train_epoch_start(self, *args, **kwargs):
        pass

    def on_train_epoch_end(self, *args, **kwargs):
        pass

    def on_train_batch_start(self, *args, **kwargs):
        pass

    def on_train_batch_end(self, *args, **kwargs):
        pass


class ModelSummary(Callback):
    pass
