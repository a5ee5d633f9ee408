from .archive import (NxsError, load_archive, load_language_model, load_model, model_archive, optim_record,  # noqa: F401
                      save_archive, save_language_model, save_model, trainer_record)
