from .pangu import Pangu
