package eu.redbean.kten.tensor.cuda.nn

import eu.redbean.kten.api.tensor.operations.TensorOperations
import eu.redbean.kten.api.tensor.operations.TensorOperationsGarbageCollector
import eu.redbean.kten.api.tensor.platform.DeviceType
import eu.redbean.kten.api.tensor.platform.PlatformProvider
import eu.redbean.kten.api.tensor.store.AbstractRawTensor
import eu.redbean.kten.tensor.tests.nn.PoolingTestsBase
import org.junit.jupiter.api.AfterEach
import org.junit.jupiter.api.BeforeAll
import org.junit.jupiter.api.BeforeEach
import org.junit.jupiter.api.TestInstance

/**
 * kten's pooling suite (the 1-D max pooling fixture of kten-testing) on the CUDA platform, one GC scope per test, as
 * CUDATensorTests runs the tensor suite.  The same fixture is what pins the oracle and the device in the Python tests
 * (tests/golden/maxpool1d_k3_s2_p1_d2_on_2x3x10_ceil.json).  Not compiled: no JDK on this box.
 */
@TestInstance(TestInstance.Lifecycle.PER_CLASS)
class CUDAPoolingTests : PoolingTestsBase() {

    private lateinit var gc: TensorOperationsGarbageCollector
    private lateinit var platformKey: String

    @BeforeAll
    @Suppress("UNCHECKED_CAST")
    fun setupDefaultOps() {
        val info = PlatformProvider.findPlatform { it.platformImplementationType == "CUDA" && it.deviceType == DeviceType.GPU }
        platformKey = info.platformKey
        PlatformProvider.registerAsDefault(platformKey, PlatformProvider.tensorOperations(platformKey) as TensorOperations<AbstractRawTensor<Any>>, info)
    }

    @BeforeEach
    fun setupGc() {
        gc = PlatformProvider.tensorOperations(platformKey).garbageCollector()
    }

    @AfterEach
    fun tearDownGc() = gc.close()
}
