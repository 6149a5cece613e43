import sys

from pagedserve_b200.main import main

sys.exit(main())
